// Device-resident records shared by the host task-graph compiler and the megakernel.
//
// Counterpart of TaskDesc / EventDesc / RuntimeConfig in the reference
// (include/mirage/persistent_kernel/runtime_header.h:219-364), re-thought for a
// statically scheduled runtime: every worker CTA owns a fixed, ordered slice of the
// task array, events are plain 64-bit counters in HBM that grow monotonically
// across launches, and there are no scheduler CTAs or queues to pop.
#pragma once
#include <stdint.h>

namespace mpk {

constexpr int kMaxDeps = 3;
constexpr int kConsumerThreads = 256;          // 8 compute warps
constexpr int kBlockThreads = kConsumerThreads + 32;  // + 1 weight-streaming warp
constexpr int kChunkRows = 16;                 // weight rows per streamed chunk, at most (one mma m-tile)
constexpr int kChunkColsMax = 2048;            // k extent of a chunk, at most (the graph compiler may settle for 1024)
constexpr int kRowPadBytes = 16;               // shared-memory row padding: conflict-free ldmatrix
constexpr int stage_bytes_for(int chunk_cols) { return kChunkRows * (chunk_cols * 2 + kRowPadBytes); }
constexpr int kPartialBytes = 8 * 1024;        // per-task partial-sum slots
constexpr int kMaxLinearTokens = 64;           // eight mma n-tiles of 8 tokens, one per compute warp
constexpr int kFp8TaskRows = 64;               // weight rows of one FP8 linear task (their scales are staged in shared memory)
constexpr int kTcSlotBytes = 16 * 1024;        // weight ring slot of graphs whose linears run on tcgen05 (1 KB multiples: swizzle atoms)
constexpr int kTmemCols = 512;                 // tensor-memory columns a worker CTA allocates (all of them: one CTA per SM)
constexpr int kTcKBlock = 64;                  // bf16 columns of one 128-byte swizzle row (an e4m3 row holds 128)
constexpr int kTcSfCols = 64;                  // tensor-memory columns kept for scale factors: 8 warps x (4 for A + 4 for B)
constexpr int kTcAccCols = kTmemCols - kTcSfCols;   // columns available to the accumulators of a task
constexpr int kTcFp8MaxTiles = 4;              // row tiles of one FP8 tcgen05 task (their scale words are staged in shared memory)

enum TaskType : uint32_t {
  TASK_NOP = 0,
  TASK_BATCH = 1,          // device-side continuous batching (prepare_next_batch)
  TASK_EMBED = 2,
  TASK_RMSNORM = 3,
  TASK_LINEAR = 4,         // weight-streaming GEMV with fused prologue/epilogue
  TASK_ATTENTION = 5,      // paged split-KV GQA decode attention
  TASK_SILU_MUL = 6,
  TASK_ARGMAX_PARTIAL = 7,
  TASK_ARGMAX_REDUCE = 8,
  TASK_ALLREDUCE = 9,      // sum the per-rank inbox slots (+ residual)
  TASK_ELEMENTWISE_ADD = 10,
  TASK_TENSOR_INIT = 11,
  TASK_QUANTIZE_FP8 = 12,  // per-token, per-128-group e4m3 quantisation (UE8M0 or float32 scales)
  TASK_MOE_ROUTING = 13,   // group-aware sigmoid top-k routing
  TASK_MOE_GEMM = 14,      // expert projections over the active experts (bf16, or e4m3 with float32 scales)
  TASK_MOE_SILU_MUL = 15,  // silu(gate) * up on [token, slot, gate | up]
  TASK_MOE_MUL_SUM_ADD = 16,  // weighted sum over expert slots + residual
  TASK_MLA_APPEND = 17,    // new [c_latent | k_pe] rows -> paged latent cache
  TASK_MLA_DECODE = 18,    // absorbed MLA decode of one (token, kv split, 16-head group): partial O + LSE
  TASK_MLA_REDUCE = 19,    // merge the splits
  TASK_SAMPLING_PARTIAL = 20,   // Gumbel-max sampling over one column range of the vocabulary
  TASK_SAMPLING_REDUCE = 21,    // merge of the column ranges (equal keys: highest index)
  TASK_ARGMAX_EXCHANGE = 22,    // argmax merge over a vocabulary sharded across ranks (pairs exchanged through the inboxes)
  TASK_AR_PUSH = 23,            // copy a column slice of a local bf16 tensor into every rank's inbox as fp32 (allreduce whose
                                // input is not produced by a bf16 linear); fields as TASK_ALLREDUCE with p[0] = the tensor
};

// prologue applied while staging the activation tile of a linear task
enum Prologue : int32_t { PRO_PLAIN = 0, PRO_RMSNORM = 1, PRO_SILU_MUL = 2 };
// epilogue of a linear task
enum Epilogue : int32_t {
  EPI_STORE = 0,        // out = bf16(acc)
  EPI_RESIDUAL = 1,     // out = bf16(acc + residual)
  EPI_PUSH_F32 = 2,     // fp32 partial rows pushed into every rank's inbox slot [my_rank] (+ counter increments)
  EPI_PUSH_LL = 3,      // {bf16 partial, 16-bit sequence} words pushed into every rank's inbox: self-validating
  EPI_SILU_PAIR = 4,    // rows interleaved [gate, gate, up, up]: out[2k + i] = bf16(silu(gate_i)) * up_i
};

// flags
constexpr uint32_t TF_SAME_X_AS_PREV = 1u << 0;    // activation tile already staged by the previous task
constexpr uint32_t TF_STREAM_AFTER_DEP = 1u << 1;  // weight operand is produced inside the graph: do not prefetch
constexpr uint32_t TF_REMOTE_TRIGGER = 1u << 2;    // trigger event lives on every rank (peer atomics)
constexpr uint32_t TF_FP8 = 1u << 3;               // linear task: e4m3 weights and activations with UE8M0 block scales
constexpr uint32_t TF_TC = 1u << 4;                // linear task on the tcgen05 path: weight tiles arrive by tensor-map TMA in the
                                                   // 128-byte-swizzled K-major layout, accumulators live in tensor memory
constexpr uint32_t TF_DEP0_REMOTE = 1u << 8;       // dependency i (bit 8 + i) is incremented by peers: system-scope acquire

struct alignas(16) TaskDesc {
  uint32_t type;
  uint32_t flags;
  int32_t dep_event[kMaxDeps];   // -1: none
  uint32_t dep_need[kMaxDeps];   // arrivals per iteration that complete the dependency
  int32_t trig_event;            // -1: none
  int32_t layer;                 // index of the layer this task was cut from (profiling / dumps)
  uint64_t p[8];                 // pointers, meaning per type
  int32_t a[28];                 // integers, meaning per type
};
constexpr int kDescVecs = 14;
static_assert(sizeof(TaskDesc) == 16 * kDescVecs, "TaskDesc must stay 224 bytes (14 x 16-byte vectors)");

// ---- TASK_LINEAR -----------------------------------------------------------
//  p[0] W [N,K] bf16 (row stride a[3])   p[1] x source   p[2] out   p[3] residual
//  p[4] gamma (PRO_RMSNORM)              p[5] inbox base (EPI_PUSH_F32, local address of slot 0)
//  a[0] n0  a[1] n1  a[2] K  a[3] ldw  a[4] ld_x  a[5] ld_out  a[6] ld_res
//  a[7] prologue  a[8] epilogue  a[9] eps bits  a[10] silu groups
//  a[11] KT (k tile of the activation)  a[12] KC (k extent of a streamed chunk)  a[13] inbox slot stride (floats)  a[14] N
//  a[18] weight rows per streamed chunk (8 or 16)
//  FP8 (TF_FP8): p[6] weight scales, p[7] activation scales, packed UE8M0 (4 exponents per uint32);
//        a[23], a[24] strides (uint32 units) of the weight scales over (row, packed k); a[25], a[26] of the
//        activation scales over (token, packed k).  K, KT, KC, ld* are in elements (= bytes).
//  a[19] 1 + index of the allreduce whose pushed partials the prologue gathers (0: none); then p[6] residual,
//        p[7] tensor that receives the reduced activations, a[20] ld residual, a[21] ld of that tensor,
//        a[22] inbox slot stride of that allreduce (words)
//  a[15] allreduce index within the iteration  a[16] allreduces per iteration  a[17] stride between the two inbox buffers (floats)
//  tcgen05 path (TF_TC): a[18] rows of one weight tile (the TMA box height, a multiple of 8, at most 128; the task's rows are
//        cut into ceil(rows / a[18]) tiles, each one 128-lane accumulator), a[12] = 64 x (k blocks of 64 columns per ring slot),
//        a[27] index of the task's tensor map (dims {64, rows of the task, K / 64}, box {64, a[18], a[12] / 64}, 128-byte swizzle)
enum { L_N0 = 0, L_N1, L_K, L_LDW, L_LDX, L_LDO, L_LDR, L_PRO, L_EPI, L_EPS, L_GROUPS, L_KT, L_KC, L_SLOT, L_N, L_ARIDX, L_NAR, L_PARSTRIDE, L_ROWS,
       L_GATHER, L_G_LDRES, L_G_LDOUT, L_G_SLOT, L_WS_S0, L_WS_S1, L_XS_S0, L_XS_S1, L_TMAP };
static_assert(L_TMAP == 27, "TaskDesc::a has 28 entries");
// ---- TASK_ATTENTION ----------------------------------------------------------
//  p[0] qkv  p[1] k_cache  p[2] v_cache  p[3] q_norm  p[4] k_norm  p[5] cos  p[6] sin  p[7] out
//  a[0] slot  a[1] kv head  a[2] chunk  a[3] num chunks  a[4] local q heads  a[5] local kv heads
//  a[6] head_dim  a[7] page_size  a[8] flags(1 qk_norm, 2 rope, 4 contiguous cache)  a[9] ld_qkv
//  a[10] ld_out  a[11] eps bits  a[12] rope table rows  a[13] cache seq (contiguous mode)
//  a[14] ticket bank offset  a[15] event of the batching task (-1: none)  a[16] its arrivals per iteration
enum { A_SLOT = 0, A_HEAD, A_CHUNK, A_NCHUNK, A_HQ, A_HKV, A_HD, A_PAGE, A_FLAGS, A_LDQKV, A_LDO, A_EPS, A_ROPE_ROWS, A_CSEQ,
       A_TICKET, A_EARLY_EV, A_EARLY_NEED };
// ---- TASK_EMBED / RMSNORM / SILU / ADD / INIT ---------------------------------
//  rows [a[0],a[1]) of the token dimension, width a[2]; p[0] in  p[1] weight/second input  p[2] out
//  a[3] ld_in  a[4] ld_out  a[5] eps bits | silu groups | vocab  a[6] ld_in2
enum { E_T0 = 0, E_T1, E_WIDTH, E_LDI, E_LDO, E_AUX, E_LDI2 };
// ---- TASK_MOE_ROUTING: p[0] logits [B, E] (zeroed after reading)  p[1] bias f32 [E]  p[2] weights f32 [B, topk]
//      p[3] routing i32 [E, ld]  p[4] active i32 [E + 1];  a[0] E  a[1] topk  a[2] groups  a[3] groups kept
//      a[4] scaling bits  a[5] ld logits  a[6] ld weights  a[7] ld routing  a[8] logits are f32
// ---- TASK_MOE_GEMM: linear-task fields (L_*) describe one expert's panel; p[0] weights [E, N, K]  p[1] x  p[2] out
//      p[4] routing  p[5] active list  p[6] weight scales f32 [E, N, K/128]  p[7] x scales f32 [rows, K/128];
//      a[M_NEXP] experts  a[M_NTOPK]  a[M_PER_SLOT] 1: x has one row per (token, slot)  a[M_LDR] ld routing
//      a[M_ESTRIDE] elements between experts
enum { M_NEXP = 19, M_NTOPK, M_PER_SLOT, M_LDR, M_ESTRIDE };
// ---- TASK_MOE_SILU_MUL: p[0] in [rows, 2I]  p[2] out [rows, I]; a[0] r0 a[1] r1 a[2] I a[3] ld in a[4] ld out a[5] rows per token
// ---- TASK_MOE_MUL_SUM_ADD: p[0] in [B, topk, H]  p[1] weights f32 [B, topk]  p[2] out  p[3] residual;
//      a[0] c0 a[1] c1 (columns) a[2] H a[3] topk a[4] ld out a[5] ld residual a[6] ld weights a[7] tokens
// ---- TASK_MLA_APPEND: p[0] c_latent_new  p[1] k_pe_new  p[2] cache [pages, page, d_k];  a[0] slot  a[1] ld c_latent
//      a[2] ld k_pe  a[3] page  a[4] d_k  a[5] d_v
// ---- TASK_MLA_DECODE: p[0] q [tokens, H * 576]  p[1] cache (paged, or contiguous [requests * kv_len, 576])
//      p[2] partial O bf16 [(token * H + head) * S + split][512]  p[3] partial LSE f32 [(token * H + head) * S + split]
//      a[0] token  a[1] split  a[2] first head  a[3] H  a[4] S  a[5] page (0: contiguous)  a[6] ld q  a[7] scale bits
//      a[8] q_len (contiguous mode)  a[9] kv_len (contiguous mode)
// ---- TASK_MLA_REDUCE: p[0] partial O  p[1] partial LSE  p[2] out [tokens, H * 512];  a[0] r0  a[1] r1 (rows = token * H + head)
//      a[2] H  a[3] S  a[4] ld out
// ---- TASK_QUANTIZE_FP8: rows [a[0],a[1]) of p[0] (bf16, width a[2], ld a[3]) -> p[1] e4m3 (ld a[4] bytes), p[2] scales;
//      a[5] 1: packed UE8M0 uint32, 0: float32; a[7], a[8] strides of the scale tensor over (token, packed k | group)
// ---- TASK_ARGMAX_PARTIAL:  p[0] logits p[1] value p[2] index  a[0] c0 a[1] c1 a[2] chunk id a[3] ld_logits a[4] ld_part
// ---- TASK_SAMPLING_PARTIAL: as TASK_ARGMAX_PARTIAL (the value is the bf16 key), plus a[6] / a[7] philox seed (low /
//                            high word), a[8] rows per reference task (the noise of row b is that of row b % a[8]),
//                            a[9] vocabulary size
// ---- TASK_ARGMAX_REDUCE:   p[0] value p[1] index p[2] out ids  a[0] num partials a[1] ld_part
// ---- TASK_SAMPLING_REDUCE:  as TASK_ARGMAX_REDUCE, but equal values go to the highest index
// ---- TASK_ARGMAX_EXCHANGE:  as TASK_ARGMAX_REDUCE, plus a[2] first column of this rank, p[5] word offset of the
//      exchange area inside an inbox buffer ([world][tokens] x {value | seq, index | seq} 64-bit words), a[L_ARIDX],
//      a[L_NAR], a[L_PARSTRIDE] as for the allreduce
// ---- TASK_ALLREDUCE:       p[0] inbox base p[1] residual (or null) p[2] out
//  a[0] c0 a[1] c1 (columns) a[2] world a[3] slot stride (floats) a[4] ld_out a[5] ld_res a[6] N
//  a[7] allreduce index  a[8] allreduces per iteration  a[9] stride between the two inbox buffers (floats)
struct BatchMeta {
  int32_t *step;
  int64_t *tokens;
  int64_t *input_tokens;
  int64_t *output_tokens;
  int32_t *prompt_lengths;
  int32_t *qo_indptr;
  int32_t *paged_kv_indptr;
  int32_t *paged_kv_indices;
  int32_t *paged_kv_last_page_len;
  int32_t *paged_kv_indices_snapshot;
  // private scheduler state owned by the handle
  int32_t *request_ids;      // [max_num_batched_requests]
  int32_t *page_queue;       // [max_num_pages]
  int32_t *sched_scalars;    // [0] page_queue_head [1] page_queue_tail [2] next_request_id
};

struct DeviceStatus {
  int32_t error;
  int32_t where;
  int32_t worker;
  int32_t task;
  int32_t all_done;
  int32_t active_tokens;
  unsigned long long iteration;   // completed launches; the running launch uses iteration + 1
  unsigned int exit_ticket;
  unsigned int pad;
  unsigned long long t_start[8];  // globaltimer at entry of CTA 0, ring indexed by iteration & 7
  unsigned long long t_end[8];    // globaltimer when the last CTA left
};

constexpr int kMaxWorld = 8;

struct KernelParams {
  const TaskDesc *tasks;
  const int32_t *worker_begin;          // [num_workers + 1]
  unsigned long long *counters;         // [num_events] local event counters
  unsigned long long *peer_counters[kMaxWorld];  // the same array on every rank (index = rank)
  float *peer_inbox[kMaxWorld];         // exchange region of every rank
  DeviceStatus *status;
  BatchMeta meta;
  float *attn_scratch;                  // split-KV partials
  unsigned int *attn_tickets;           // [max_requests * kv_heads] per attention layer slot
  uint64_t *profiler;
  uint64_t profiler_entries;
  long long eos_token_id;
  int32_t num_workers;
  int32_t test_mode;
  int32_t world_size, rank;
  int32_t max_seq_length, max_num_batched_requests, max_num_batched_tokens, max_num_pages, page_size;
  int32_t total_num_requests;
  int32_t num_stages;                   // weight pipeline depth
  int32_t stage_bytes;                  // bytes of one stage: 16 rows x (chunk columns x 2 + 16)
  uint32_t poll_sleep_ns;               // back-off between two polls of an event counter (0: none)
  int32_t quiet_streaming;              // hold the weight stream back while attention tasks run
  int32_t kv_l2_prefetch;               // streaming warp prefetches attention K/V rows into L2
  int32_t max_inflight;                 // chunks the streamer keeps in flight (<= num_stages)
  int32_t ll_row_words;                 // words of one token row in a rank's inbox slot when all fused allreduces have the same
                                        // width (0: they differ): the batching task clears rows that go idle (see ll_seq)
  int32_t ll_buffer_words;              // words between the two inbox buffers
  int32_t tp_extensions;                // batch-1 graphs of several ranks: run the instantiation with the argmax exchange and the
                                        // all-ranks-in-flight allreduce prologue (set when the graph holds an exchange task)
  int32_t general_kernel;               // host side: launch the instantiation with FP8 and > 8-token linear tasks
  int32_t x_tile_bytes;                 // bytes reserved for the activation tile
  uint32_t spin_limit;                  // polls before a wait gives up
  const void *tmaps;                    // array of 128-byte tensor maps (one per tcgen05 linear task), 64-byte aligned
  int32_t use_tmem;                     // the graph has tcgen05 tasks: every worker CTA allocates tensor memory
  int32_t tc_tokens;                    // token rows of the activation operand tile (batched tokens rounded up to 16)
  int32_t meta_static;                  // the batch description is the caller's and final at launch (test mode, online_notoken):
                                        // the graph has no batching task
};

}  // namespace mpk
