/*
 * mpk_b200.h -- C ABI of libmpk_b200.so, a B200 (sm_100a) decode megakernel that
 * stands in for the Mirage Persistent Kernel (MPK) runtime of mirage-project/mirage.
 *
 * The reference binds its runtime through a CPython extension generated at
 * compile() time ("__mirage_launcher", python/mirage/mpk/persistent_kernel.py:21-167)
 * that wraps four extern "C" functions taking std::vector arguments
 * (include/mirage/persistent_kernel/persistent_kernel.cuh:1167-1603) and keeps its
 * state in one process-global RuntimeConfig (:1151).  This header is the
 * equivalent boundary as a true C ABI: plain pointers and sizes, an opaque handle
 * instead of a global, int status codes instead of exit()/abort().
 *
 * Every function returns MPK_OK (0) or a negative mpk_error; mpk_last_error()
 * gives the message.  Nothing here allocates or touches the device before
 * mpk_compile(), except where noted.
 */
#ifndef MPK_B200_H
#define MPK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mpk_handle mpk_handle;

typedef enum {
  MPK_OK = 0,
  MPK_ERR_INVALID = -1,      /* bad argument / malformed graph                */
  MPK_ERR_CUDA = -2,         /* a CUDA runtime call failed                    */
  MPK_ERR_UNSUPPORTED = -3,  /* shape or feature outside what the kernel does */
  MPK_ERR_TIMEOUT = -4,      /* a bounded device-side wait expired            */
  MPK_ERR_STATE = -5,        /* call out of order (e.g. launch before compile)*/
  MPK_ERR_DEADLOCK = -6      /* host simulation of the task graph got stuck   */
} mpk_error;

/* dtype codes follow python/mirage/_cython/CCore.pxd (DT_* enum) only in spirit:
 * the values are this library's own. */
typedef enum {
  MPK_BF16 = 0, MPK_F16 = 1, MPK_F32 = 2, MPK_I32 = 3, MPK_I64 = 4,
  MPK_F8E4M3 = 5, MPK_U32 = 6, MPK_U8 = 7, MPK_U64 = 8, MPK_I16 = 9
} mpk_dtype;

/* execution modes, python/mirage/mpk/persistent_kernel.py:169 */
typedef enum { MPK_MODE_OFFLINE = 0, MPK_MODE_ONLINE_NOTOKEN = 1 } mpk_mode;

/* io_category of PersistentKernel.new_tensor, persistent_kernel.py:546-568 */
typedef enum { MPK_IO_CUDA = 0, MPK_IO_SYMMETRIC = 1 } mpk_io_category;

/* Layer operators: one per PersistentKernel.*_layer method on the decode path
 * (python/mirage/mpk/persistent_kernel.py, line of each method in the comment). */
typedef enum {
  MPK_OP_EMBED = 1,             /* embed_layer              :586  in: ids, table        out: y            params: [input_source]          */
  MPK_OP_RMSNORM = 2,           /* rmsnorm_layer            :609  in: x, gamma          out: y                                            */
  MPK_OP_RMSNORM_LINEAR = 3,    /* rmsnorm_linear_layer     :627  in: x, gamma, W       out: y                                            */
  MPK_OP_LINEAR = 4,            /* linear_layer             :1731 in: x, W              out: y                                            */
  MPK_OP_LINEAR_RESIDUAL = 5,   /* linear_with_residual_layer :1762 in: x, W, residual  out: y            params: [enable_residual]       */
  MPK_OP_SPLITK_LINEAR = 6,     /* splitk_linear_layer      :1706 in: x, W              out: y (y += x W^T)                               */
  MPK_OP_ATTENTION = 7,         /* attention_layer          :648  in: qkv,k,v,qn,kn,cos,sin out: o       params: [hq, hkv, qk_norm, rope] */
  MPK_OP_PAGED_ATTENTION = 8,   /* paged_attention_layer    :785  same tensors                          params: [hq, hkv, qk_norm, rope, max_seq, page] */
  MPK_OP_SILU_MUL = 9,          /* silu_mul_layer           :1826 in: mid               out: act   (grid.x = interleave groups)           */
  MPK_OP_ALLREDUCE = 10,        /* allreduce_layer          :1801 in: x, buffer         out: y            params: [world, rank]           */
  MPK_OP_ARGMAX_PARTIAL = 11,   /* argmax_partial_layer     :1916 in: logits            out: value, index (grid.x = chunks)               */
  MPK_OP_ARGMAX_REDUCE = 12,    /* argmax_reduce_layer      :1941 in: value, index      out: token ids                                    */
  MPK_OP_ELEMENTWISE_ADD = 13,  /* elementwise_add_layer    :1863 in: a, b              out: y                                            */
  MPK_OP_TENSOR_INIT = 14,      /* tensor_init_layer        :1365 in: t (zero-filled)                                                     */
  MPK_OP_QUANTIZE_FP8 = 15,     /* quantize_fp8_layer       :1561 in: x               out: x_fp8, scale  params: [scale_ue8m0]            */
  MPK_OP_LINEAR_FP8 = 16,       /* linear_fp8_layer         :1584 in: x_fp8, x_scale, w_fp8, w_scale   out: y                            */
  MPK_OP_LINEAR_FP8_RESIDUAL = 17, /* linear_fp8_with_residual_layer :1611 in: x_fp8, x_scale, w_fp8, w_scale, residual  out: y           */
  MPK_OP_MOE_TOPK_SIGMOID = 18, /* moe_topk_sigmoid_routing_layer :1408 in: logits, bias  out: topk_weight, routing_indices, mask  params: [num_groups, topk_group, scaling_bits] */
  MPK_OP_MOE_W13_LINEAR = 19,   /* moe_w13_linear_layer     :1444 in: x, w, routing_indices, mask         out: y [B, topk, 2I]           */
  MPK_OP_MOE_W2_LINEAR = 20,    /* moe_w2_linear_layer      :1652 in: x [B, topk, I], w, routing_indices, mask  out: y [B, topk, H]      */
  MPK_OP_MOE_W13_FP8 = 21,      /* moe_w13_fp8_layer        :1475 in: x_fp8, x_scale, w_fp8, w_scale, routing_indices, mask  out: y      */
  MPK_OP_MOE_W2_FP8 = 22,       /* moe_w2_fp8_layer         :1518 in: x_fp8, x_scale, w_fp8, w_scale, routing_indices, mask  out: y      */
  MPK_OP_MOE_SILU_MUL = 23,     /* moe_silu_mul_layer       :1636 in: mid [B, topk, 2I]    out: act [B, topk, I]                         */
  MPK_OP_MOE_MUL_SUM_ADD = 24,  /* moe_mul_sum_add_layer    :1683 in: x [B, topk, H], topk_weight, residual   out: y [B, H]              */
  MPK_OP_MLA_KV_GATHER = 25,    /* mla_kv_gather_layer      :995  in: c_latent_new, k_pe_new  inout: paged_cache  (contiguous_kv unused)  params: [d_k, d_v, page_size] */
  MPK_OP_MLA_DECODE = 26,       /* mla_mtp_decode_layer     :1165 (and mla_decode_layer :1045, _tp2/4/8 :1307-1355) in: q, cache  out: partial_o, partial_lse
                                   params: [num_heads, q_len, kv_len, num_splits, scale_bits, page_size (0: cache is contiguous [requests * kv_len, 576])] */
  MPK_OP_MLA_REDUCE = 27,       /* mla_mtp_reduce_layer     :1195 (and mla_reduce_layer :1077) in: partial_o, partial_lse  out: o  params: [num_heads, num_splits] */
  /* sampling_sm100_layer :1968 (Gumbel-max sampling, tasks/common/sampling.cuh:158-226) is split like argmax into
   * per-column-range partials and one merge.  key = bf16(logit) + bf16(gumbel(philox4x32-10(seed, subsequence,
   * offset 0))) in bf16, largest key wins, equal keys go to the HIGHEST index. */
  MPK_OP_SAMPLING_PARTIAL = 28, /* in: logits [B, V] bf16  out: part_key [B, >= grid.x] bf16, part_index int64  params: [seed, rows_per_task] */
  MPK_OP_SAMPLING_REDUCE = 29,  /* in: part_key, part_index  out: ids [B, 1] int64 */
  /* No reference counterpart (the reference keeps the whole lm_head on every rank).  Merge of argmax partials when the
   * vocabulary is sharded over the tensor-parallel ranks: every rank merges its own partials, adds params[0] to the
   * winning column index, pushes {value, index} into every peer's exchange region, gathers the ranks' pairs and writes
   * the global winner (largest value, lowest index on ties): all ranks write the same ids. */
  MPK_OP_ARGMAX_EXCHANGE = 30,  /* in: value, index (local columns)  out: token ids   params: [first column of this rank] */
  MPK_OP_MOE_TOPK_SOFTMAX = 31  /* moe_topk_softmax_routing_layer :1385 in: logits  out: topk_weight, routing_indices, mask
                                   (softmax over the experts, top-k by value with ties to the lower index, weights renormalised
                                   over the selected experts; the logits are left as they are)  params: optional [first, end]
                                   of the experts this rank runs */
} mpk_op;

/* Constructor arguments of PersistentKernel (persistent_kernel.py:349-369) plus the
 * meta tensors it hands to init_func (:2494-2506).  All pointers are DEVICE
 * pointers borrowed from the caller for the life of the handle; they may be NULL
 * in test mode. */
typedef struct {
  int32_t mode;                      /* mpk_mode */
  int32_t test_mode;                 /* run the task graph once per launch, no batching */
  int32_t dry_run;                   /* build and check the task graph only: no CUDA call at all */
  int32_t device;                    /* CUDA device ordinal */
  int32_t world_size, rank;          /* tensor-parallel group */
  int32_t num_workers;               /* worker CTAs; <= 0: one per SM */
  int32_t max_seq_length;
  int32_t max_num_batched_requests;
  int32_t max_num_batched_tokens;
  int32_t max_num_pages;
  int32_t page_size;
  int32_t total_num_requests;
  int32_t reserved0;
  int64_t eos_token_id;
  int32_t *step;                     /* [total_num_requests]          */
  int64_t *tokens;                   /* [total_num_requests, max_seq] */
  int64_t *input_tokens;             /* [max_num_batched_tokens]      */
  int64_t *output_tokens;            /* [max_num_batched_tokens]      */
  int32_t *num_new_tokens;           /* [total_num_requests]          */
  int32_t *prompt_lengths;           /* [total_num_requests]          */
  int32_t *qo_indptr;                /* [max_num_batched_requests+1]  */
  int32_t *paged_kv_indptr;          /* [max_num_batched_requests+1]  */
  int32_t *paged_kv_indices;         /* [max_num_pages]               */
  int32_t *paged_kv_last_page_len;   /* [max_num_batched_requests]    */
  int32_t *paged_kv_indices_snapshot;/* [max_num_pages]               */
  uint64_t *profiler_buffer;         /* optional: 8 uint64 per task, this library's own record (NOT the reference's (tag, globaltimer) stream
                                        of include/mirage/persistent_kernel/profiler.h:90-157): [0] wait begin, [1] dependencies met,
                                        [2] task end (globaltimer ns), [3] worker << 40 | event << 8 | task type, [4..7] phase stamps
                                        whose meaning depends on the task type; mirage_b200/profiler.py converts to a Chrome trace */
  uint64_t profiler_entries;
} mpk_config;

/* What the device reported after the most recent launch. */
typedef struct {
  int32_t error;          /* 0, or MPK_ERR_TIMEOUT                             */
  int32_t where;          /* 1 dependency wait, 2 weight pipeline, 3 peer wait */
  int32_t worker;         /* CTA that gave up                                  */
  int32_t task;           /* index of its task                                 */
  int32_t all_done;       /* offline mode: no request left to run              */
  int32_t active_tokens;  /* tokens in the last batch                          */
  uint64_t iteration;     /* launches completed since the last reset           */
} mpk_status;

/* replaces init_persistent_kernel's config parsing, persistent_kernel.cuh:1173-1222 */
int mpk_create(const mpk_config *cfg, mpk_handle **out);
/* replaces finalize_persistent_kernel, persistent_kernel.cuh:1557-1603 (and also frees new_tensor storage) */
int mpk_destroy(mpk_handle *h);
const char *mpk_last_error(const mpk_handle *h);

/* Graph::attach_torch_tensor, src/kernel/graph.cc:338-372: borrow a device pointer.  Returns tensor id >= 0. */
int mpk_attach_tensor(mpk_handle *h, const char *name, void *device_ptr, int dtype,
                      int ndim, const int64_t *dims, const int64_t *strides);
/* Graph::attach_cuda_tensor / attach_nvshmem_tensor, graph.cc:374-400: storage owned by the handle,
 * allocated (zero-filled) by mpk_compile. */
int mpk_new_tensor(mpk_handle *h, const char *name, int dtype, int ndim,
                   const int64_t *dims, const int64_t *strides, int io_category);
/* Graph::fuse_tensors graph.cc:402-419 / shuffle_tensors :421-437 (dim 0 only).  The result is a new
 * handle-owned tensor filled at compile time by interleaving `num_groups` equal row blocks of the inputs. */
int mpk_shuffle_tensors(mpk_handle *h, const char *name, const int *tensor_ids, int n, int num_groups);
int mpk_fuse_tensors(mpk_handle *h, const char *name, const int *tensor_ids, int n, int num_groups);

/* Graph::register_task, src/kernel/graph.cc:439-853: append one layer.  tensor_ids lists inputs then outputs
 * in the order of the mpk_op comment; -1 stands for an absent optional tensor.  grid is the reference's
 * grid_dim, used as a partitioning hint.  Returns the layer index. */
int mpk_add_layer(mpk_handle *h, int op, const int *tensor_ids, int n_tensors,
                  const int grid[3], const int64_t *params, int n_params);

/* Graph::generate_task_graph + init_persistent_kernel, src/kernel/runtime.cc:1872-1906 and
 * persistent_kernel.cuh:1173-1470: fold norm/activation layers into their consumers, cut layers into
 * tasks, derive events, check the graph by host simulation, allocate and upload. */
int mpk_compile(mpk_handle *h);

/* Tensor-parallel set-up (stands in for nvshmem_malloc + teams, persistent_kernel.cuh:1105-1122,1225-1282).
 * After mpk_compile every rank exports the 64-byte CUDA IPC handle of its exchange region, the caller
 * moves the handles between processes, and each rank imports all peers before the first launch. */
int mpk_comm_export(mpk_handle *h, void *ipc_handle_64B);
int mpk_comm_import(mpk_handle *h, int peer_rank, const void *ipc_handle_64B);
/* Same-process variant for tests: peers are handles living in one process (one per device). */
int mpk_comm_link_local(mpk_handle *h, int peer_rank, mpk_handle *peer);

/* init_request_resources / init_kernel, persistent_kernel.cuh:142-169: reset scheduler state (steps,
 * page ring, request slots) and event counters.  Called implicitly by the first launch. */
int mpk_reset(mpk_handle *h, void *cuda_stream);
/* launch_persistent_kernel, persistent_kernel.cuh:1474-1555: enqueue `num_steps` megakernel launches
 * (one decode iteration each) on the stream.  Asynchronous. */
int mpk_launch(mpk_handle *h, void *cuda_stream, int num_steps);
/* Synchronise the stream and read the device status block. */
int mpk_sync_status(mpk_handle *h, void *cuda_stream, mpk_status *out);

/* Introspection. */
int mpk_tensor_ptr(mpk_handle *h, int tensor_id, void **device_ptr, uint64_t *bytes);
int mpk_graph_info(mpk_handle *h, int *num_tasks, int *num_events, int *num_workers, int *num_layers_folded);
/* Text dump of the task graph (what generate_task_graph returns as "json_file"); returns bytes needed. */
int64_t mpk_dump_task_graph(mpk_handle *h, char *buf, int64_t buf_bytes);
/* Weight bytes one launch streams from HBM (sum over linear tasks), for roofline accounting. */
int64_t mpk_weight_bytes_per_step(mpk_handle *h);

/* No counterpart in the reference.  Split-KV paged GQA decode attention (one new token per request, head_dim
 * 128, no QK-norm / RoPE: q, k, v are used as given) for callers that must not allocate device memory at call
 * time -- e.g. while a stream is being captured, or under a memory pool that owns the whole device.  It needs no
 * handle and calls no cudaMalloc / cudaFree: the split-KV partials and arrival tickets live in a 4 MiB array
 * inside the library image (resident on every GPU that loads the library until the process exits).
 *   qkv   [num_requests, ld_qkv] bf16, per kv head [q x (num_q_heads/num_kv_heads) | k | v], 128 wide each
 *   k_cache / v_cache [pages, page_size, num_kv_heads, 128] bf16; the new k/v row is appended at position
 *         seq_len-1 of each request (kv_* arrays describe the sequences INCLUDING that position)
 *   out   [num_requests, ld_out] bf16, num_q_heads * 128 wide
 * A request whose kv_* entries describe an empty sequence (no page) gets a zero output row and appends nothing.
 * Preconditions checked before anything is launched (MPK_ERR_INVALID): ld_qkv >= num_kv_heads * (G + 2) * 128,
 * ld_out >= num_q_heads * 128, both strides multiples of 4 elements, the four bf16 pointers 8-byte aligned
 * (the kernel moves rows as 8-byte vectors), the index arrays 4-byte aligned.  Not checkable here and left to
 * the caller: every pointer must belong to the CURRENT device, v_cache has k_cache's shape, kv_indptr holds
 * num_requests + 1 entries and kv_last_page_len num_requests.
 * Limits: num_requests * num_kv_heads <= 4096 and 16 KiB + num_requests * num_q_heads * num_chunks * 520 B <= 4 MiB;
 * larger problems are refused with MPK_ERR_UNSUPPORTED and a message in `err`.
 * The first call on a device resolves the array's device address; make it before any stream capture.
 * All calls share the array: calls that may overlap on the GPU race; keep them on one stream. */
int mpk_paged_decode_attention_noalloc(const void *qkv, void *k_cache, void *v_cache, void *out,
                                       const int32_t *kv_indptr, const int32_t *kv_indices,
                                       const int32_t *kv_last_page_len, int num_requests, int num_q_heads,
                                       int num_kv_heads, int page_size, int64_t ld_qkv, int64_t ld_out,
                                       int num_chunks, void *cuda_stream, char *err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif /* MPK_B200_H */
