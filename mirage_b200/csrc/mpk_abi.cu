// C ABI of libmpk_b200.so (declared in include/mpk_b200.h).
//
// Host-side counterpart of init/launch/finalize_persistent_kernel in the reference
// (include/mirage/persistent_kernel/persistent_kernel.cuh:1167-1603): owns the tensors the
// graph allocates, compiles the layer list into a static task schedule, uploads it and
// launches the pre-built megakernel once per decode iteration.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/mpk_b200.h"
#include "runtime_types.h"
#include "task_graph.h"

extern "C" int mpk_kernel_smem_bytes(int num_stages, int stage_bytes, int x_tile_bytes);
extern "C" int mpk_kernel_prepare(int smem_bytes);
extern "C" int mpk_kernel_launch(const mpk::KernelParams *params, int smem_bytes, void *stream);
extern "C" int mpk_shuffle_rows_launch(void *dst, const void *const *srcs_dev, const int64_t *rows_per_group_dev,
                                       const int64_t *prefix_rows_dev, int n, int64_t group_rows_total,
                                       int64_t row_bytes, int64_t total_rows, void *stream);

using namespace mpk;

struct mpk_handle {
  mpk_config cfg;
  std::vector<TensorInfo> tensors;
  std::vector<LayerInfo> layers;
  CompiledGraph graph;
  std::string error;
  bool compiled = false;
  bool needs_reset = true;
  bool reset_after_error = false;     // needs_reset was set by a device timeout (not by compile)
  int num_sms = 148;
  int smem_bytes = 0;
  // device allocations
  std::vector<void *> owned;          // everything to cudaFree
  TaskDesc *d_tasks = nullptr;
  int32_t *d_worker_begin = nullptr;
  DeviceStatus *d_status = nullptr;
  uint8_t *comm = nullptr;            // exchange region: [event counters | inbox buffer 0 | inbox buffer 1]
  uint64_t comm_bytes = 0;
  uint64_t counters_bytes = 0;
  void *peer_comm[kMaxWorld] = {};
  bool peer_opened[kMaxWorld] = {};
  int32_t *d_request_ids = nullptr, *d_page_queue = nullptr, *d_sched = nullptr;
  float *d_attn_scratch = nullptr;
  unsigned int *d_attn_tickets = nullptr;
  void *d_tmaps = nullptr;            // tensor maps of the tcgen05 linear tasks
  KernelParams params;
  uint64_t fake_ptr = 0x100000;       // dry-run address allocator
};

namespace {

int elt_bytes(int dtype) {
  switch (dtype) {
    case MPK_BF16: case MPK_F16: case MPK_I16: return 2;
    case MPK_F32: case MPK_I32: case MPK_U32: return 4;
    case MPK_I64: case MPK_U64: return 8;
    default: return 1;
  }
}

int set_err(mpk_handle *h, int code, const std::string &msg) {
  if (h) h->error = msg;
  return code;
}

#define CU(call)                                                                                      \
  do {                                                                                                \
    cudaError_t e__ = (call);                                                                         \
    if (e__ != cudaSuccess)                                                                           \
      return set_err(h, MPK_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__));          \
  } while (0)

int dev_alloc(mpk_handle *h, void **out, uint64_t bytes, bool zero = true) {
  bytes = std::max<uint64_t>(bytes, 16);
  if (h->cfg.dry_run) {
    *out = reinterpret_cast<void *>(h->fake_ptr);
    h->fake_ptr += (bytes + 255) / 256 * 256;
    return MPK_OK;
  }
  CU(cudaMalloc(out, bytes));
  h->owned.push_back(*out);
  if (zero) CU(cudaMemset(*out, 0, bytes));
  return MPK_OK;
}

uint64_t tensor_bytes(const TensorInfo &t) {
  // span of a strided tensor
  uint64_t last = 0;
  for (size_t i = 0; i < t.dims.size(); ++i) {
    if (t.dims[i] <= 0) return 0;
    last += (uint64_t)(t.dims[i] - 1) * (uint64_t)t.strides[i];
  }
  return (last + 1) * elt_bytes(t.dtype);
}

int add_tensor(mpk_handle *h, const char *name, void *ptr, int dtype, int ndim, const int64_t *dims,
               const int64_t *strides, int owner) {
  if (!h) return MPK_ERR_INVALID;
  if (h->compiled) return set_err(h, MPK_ERR_STATE, "graph already compiled");
  if (ndim <= 0 || ndim > 6 || !dims) return set_err(h, MPK_ERR_INVALID, "bad tensor rank");
  TensorInfo t;
  t.name = name ? name : "";
  t.ptr = ptr;
  t.dtype = dtype;
  t.dims.assign(dims, dims + ndim);
  if (strides) {
    t.strides.assign(strides, strides + ndim);
  } else {
    t.strides.assign(ndim, 1);
    for (int i = ndim - 2; i >= 0; --i) t.strides[i] = t.strides[i + 1] * t.dims[i + 1];
  }
  t.owner = owner;
  t.bytes = tensor_bytes(t);
  h->tensors.push_back(t);
  return (int)h->tensors.size() - 1;
}

// Encode the tensor maps of the tcgen05 linear tasks and upload them.  The driver's encoder is reached through
// the runtime (cudaGetDriverEntryPoint), so the library does not link against libcuda.
int upload_tensor_maps(mpk_handle *h) {
  const std::vector<TmapSpec> &specs = h->graph.tmaps;
  if (specs.empty() || h->cfg.dry_run) return MPK_OK;
  typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  CU(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  if (!fn || qres != cudaDriverEntryPointSuccess)
    return set_err(h, MPK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  encode_fn encode = reinterpret_cast<encode_fn>(fn);
  static_assert(sizeof(CUtensorMap) == 128, "tensor maps are indexed as 128-byte records on the device");
  std::vector<CUtensorMap> maps(specs.size());
  for (size_t i = 0; i < specs.size(); ++i) {
    const TmapSpec &m = specs[i];
    const cuuint32_t inner = (cuuint32_t)(128 / m.elt_bytes);   // elements of one 128-byte swizzle row
    if ((m.base & 15u) != 0 || (m.ld_bytes & 15) != 0)
      return set_err(h, MPK_ERR_UNSUPPORTED, "linear weights on the tensor path need 16-byte aligned rows");
    const cuuint64_t dims[3] = {inner, (cuuint64_t)m.rows, (cuuint64_t)m.kblocks};
    const cuuint64_t strides[2] = {(cuuint64_t)m.ld_bytes, 128};   // bytes, dimensions 1 and 2
    const cuuint32_t box[3] = {inner, (cuuint32_t)m.box_rows, (cuuint32_t)m.box_kblocks};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = encode(&maps[i], m.elt_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                              reinterpret_cast<void *>(m.base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return set_err(h, MPK_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r) + " (rows " +
                                          std::to_string(m.rows) + ", row bytes " + std::to_string(m.ld_bytes) + ", box " +
                                          std::to_string(m.box_rows) + " x " + std::to_string(m.box_kblocks) + ")");
  }
  int rc = dev_alloc(h, &h->d_tmaps, maps.size() * sizeof(CUtensorMap), false);
  if (rc) return rc;
  CU(cudaMemcpy(h->d_tmaps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice));
  return MPK_OK;
}

}  // namespace

extern "C" {

int mpk_create(const mpk_config *cfg, mpk_handle **out) {
  if (!cfg || !out) return MPK_ERR_INVALID;
  mpk_handle *h = new mpk_handle();
  h->cfg = *cfg;
  *out = h;
  if (cfg->world_size < 1 || cfg->world_size > kMaxWorld || cfg->rank < 0 || cfg->rank >= cfg->world_size)
    return set_err(h, MPK_ERR_INVALID, "world_size must be 1..8 and 0 <= rank < world_size");
  if (cfg->max_num_batched_tokens < 1 || cfg->max_num_batched_requests < 1)
    return set_err(h, MPK_ERR_INVALID, "max_num_batched_tokens/requests must be >= 1");
  if (!cfg->test_mode) {
    if (cfg->page_size < 1 || cfg->max_num_pages < 1 || cfg->max_seq_length < 1)
      return set_err(h, MPK_ERR_INVALID, "page_size, max_num_pages, max_seq_length must be >= 1");
    const bool online = cfg->mode == MPK_MODE_ONLINE_NOTOKEN;
    if (!cfg->dry_run && (!cfg->input_tokens || !cfg->qo_indptr || !cfg->paged_kv_indptr || !cfg->paged_kv_indices ||
                          !cfg->paged_kv_last_page_len))
      return set_err(h, MPK_ERR_INVALID, "the batch description (input_tokens, qo_indptr, paged_kv_*) is required");
    if (!cfg->dry_run && !online && (!cfg->step || !cfg->tokens || !cfg->output_tokens || !cfg->prompt_lengths))
      return set_err(h, MPK_ERR_INVALID, "offline mode needs all meta tensors");
    if (cfg->max_num_batched_requests > 1024)
      return set_err(h, MPK_ERR_UNSUPPORTED, "max_num_batched_requests above 1024");
  }
  if (!cfg->dry_run) {
    cudaError_t e = cudaSetDevice(cfg->device);
    if (e != cudaSuccess) return set_err(h, MPK_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, cfg->device);
    if (e != cudaSuccess) return set_err(h, MPK_ERR_CUDA, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
    if (prop.major != 10)
      return set_err(h, MPK_ERR_UNSUPPORTED, "libmpk_b200 is built for sm_100a only; device is sm_" +
                                                 std::to_string(prop.major * 10 + prop.minor));
    h->num_sms = prop.multiProcessorCount;
  }
  return MPK_OK;
}

int mpk_destroy(mpk_handle *h) {
  if (!h) return MPK_ERR_INVALID;
  if (!h->cfg.dry_run) {
    cudaSetDevice(h->cfg.device);
    for (int r = 0; r < kMaxWorld; ++r)
      if (h->peer_opened[r]) cudaIpcCloseMemHandle(h->peer_comm[r]);
    for (void *p : h->owned) cudaFree(p);
  }
  delete h;
  return MPK_OK;
}

const char *mpk_last_error(const mpk_handle *h) { return h ? h->error.c_str() : "null handle"; }

int mpk_attach_tensor(mpk_handle *h, const char *name, void *device_ptr, int dtype, int ndim, const int64_t *dims,
                      const int64_t *strides) {
  if (h && !device_ptr && !h->cfg.dry_run) return set_err(h, MPK_ERR_INVALID, "attach_tensor: null pointer");
  return add_tensor(h, name, device_ptr, dtype, ndim, dims, strides, 0);
}

int mpk_new_tensor(mpk_handle *h, const char *name, int dtype, int ndim, const int64_t *dims, const int64_t *strides,
                   int io_category) {
  return add_tensor(h, name, nullptr, dtype, ndim, dims, strides, io_category == MPK_IO_SYMMETRIC ? 2 : 1);
}

static int shuffle_common(mpk_handle *h, const char *name, const int *ids, int n, int num_groups) {
  if (!h || !ids || n < 1 || num_groups < 1) return set_err(h, MPK_ERR_INVALID, "shuffle_tensors: bad arguments");
  int64_t rows = 0;
  for (int i = 0; i < n; ++i) {
    if (ids[i] < 0 || ids[i] >= (int)h->tensors.size()) return set_err(h, MPK_ERR_INVALID, "shuffle_tensors: bad id");
    const TensorInfo &t = h->tensors[ids[i]];
    const TensorInfo &t0 = h->tensors[ids[0]];
    if (t.dims.size() != 2 || t.dim(1) != t0.dim(1) || t.dtype != t0.dtype || t.strides[1] != 1 ||
        t.strides[0] != t.dim(1))
      return set_err(h, MPK_ERR_UNSUPPORTED, "shuffle_tensors: inputs must be contiguous 2-D with equal width");
    if (t.dim(0) % num_groups != 0) return set_err(h, MPK_ERR_INVALID, "shuffle_tensors: rows not divisible by groups");
    rows += t.dim(0);
  }
  const int64_t dims[2] = {rows, h->tensors[ids[0]].dim(1)};
  const int id = add_tensor(h, name, nullptr, h->tensors[ids[0]].dtype, 2, dims, nullptr, 3);
  if (id < 0) return id;
  h->tensors[id].shuffle_src.assign(ids, ids + n);
  h->tensors[id].shuffle_groups = num_groups;
  return id;
}

int mpk_shuffle_tensors(mpk_handle *h, const char *name, const int *tensor_ids, int n, int num_groups) {
  return shuffle_common(h, name, tensor_ids, n, num_groups);
}
int mpk_fuse_tensors(mpk_handle *h, const char *name, const int *tensor_ids, int n, int num_groups) {
  // The reference's fused tensor is a virtual concat addressed group by group
  // (src/kernel/graph.cc:402-419); materialising the same interleaving gives identical contents.
  return shuffle_common(h, name, tensor_ids, n, num_groups);
}

int mpk_add_layer(mpk_handle *h, int op, const int *tensor_ids, int n_tensors, const int grid[3],
                  const int64_t *params, int n_params) {
  if (!h) return MPK_ERR_INVALID;
  if (h->compiled) return set_err(h, MPK_ERR_STATE, "graph already compiled");
  if (!tensor_ids || n_tensors < 1) return set_err(h, MPK_ERR_INVALID, "add_layer: no tensors");
  LayerInfo l;
  l.op = op;
  l.t.assign(tensor_ids, tensor_ids + n_tensors);
  for (int t : l.t)
    if (t < -1 || t >= (int)h->tensors.size()) return set_err(h, MPK_ERR_INVALID, "add_layer: bad tensor id");
  if (grid) for (int i = 0; i < 3; ++i) l.grid[i] = grid[i];
  if (params && n_params > 0) l.params.assign(params, params + n_params);
  h->layers.push_back(l);
  return (int)h->layers.size() - 1;
}

int mpk_compile(mpk_handle *h) {
  if (!h) return MPK_ERR_INVALID;
  if (h->compiled) return set_err(h, MPK_ERR_STATE, "already compiled");
  const mpk_config &cfg = h->cfg;
  const bool dry = cfg.dry_run != 0;
  if (!dry) CU(cudaSetDevice(cfg.device));
  // 1. storage for handle-owned tensors
  for (auto &t : h->tensors) {
    if (t.owner == 0) continue;
    int rc = dev_alloc(h, &t.ptr, t.bytes);
    if (rc) return rc;
  }
  // 2. materialise shuffled tensors (after the compiler chose the interleave of [gate | up] weights whose
  //    activation it applies in the linear's epilogue)
  plan_silu_epilogue(cfg, &h->tensors, &h->layers);
  for (auto &t : h->tensors) {
    if (t.owner != 3 || dry) continue;
    const int n = (int)t.shuffle_src.size();
    std::vector<const void *> srcs(n);
    std::vector<int64_t> rpg(n), prefix(n + 1, 0);
    for (int i = 0; i < n; ++i) {
      const TensorInfo &s = h->tensors[t.shuffle_src[i]];
      srcs[i] = s.ptr;
      rpg[i] = s.dim(0) / t.shuffle_groups;
      prefix[i + 1] = prefix[i] + rpg[i];
    }
    const int64_t row_bytes = t.dim(1) * elt_bytes(t.dtype);
    if (row_bytes % 4 != 0) return set_err(h, MPK_ERR_UNSUPPORTED, "shuffle_tensors: row bytes must be a multiple of 4");
    void *d_srcs, *d_rpg, *d_prefix;
    CU(cudaMalloc(&d_srcs, n * sizeof(void *)));
    CU(cudaMalloc(&d_rpg, n * 8));
    CU(cudaMalloc(&d_prefix, (n + 1) * 8));
    CU(cudaMemcpy(d_srcs, srcs.data(), n * sizeof(void *), cudaMemcpyHostToDevice));
    CU(cudaMemcpy(d_rpg, rpg.data(), n * 8, cudaMemcpyHostToDevice));
    CU(cudaMemcpy(d_prefix, prefix.data(), (n + 1) * 8, cudaMemcpyHostToDevice));
    int rc = mpk_shuffle_rows_launch(t.ptr, (const void *const *)d_srcs, (const int64_t *)d_rpg,
                                     (const int64_t *)d_prefix, n, prefix[n], row_bytes, t.dim(0), nullptr);
    if (rc) return set_err(h, MPK_ERR_CUDA, "shuffle kernel launch failed");
    CU(cudaDeviceSynchronize());
    cudaFree(d_srcs); cudaFree(d_rpg); cudaFree(d_prefix);
  }
  // 3. storage ids: tensors whose byte ranges [ptr, ptr + bytes) overlap -- the same base pointer, or views and slices
  //    of one allocation -- share a storage, so that layers touching them are ordered against each other; the batch
  //    meta tensors map to the two reserved ids so that layers touching them are ordered against the batching task
  {
    int next = 2;
    auto meta_in = [&](void *p) {
      return p && (p == cfg.input_tokens || p == cfg.step || p == cfg.tokens || p == cfg.qo_indptr ||
                   p == cfg.paged_kv_indptr || p == cfg.paged_kv_indices || p == cfg.paged_kv_last_page_len ||
                   p == cfg.prompt_lengths || p == cfg.num_new_tokens);
    };
    const bool batched = !cfg.test_mode && cfg.mode != MPK_MODE_ONLINE_NOTOKEN;
    std::vector<size_t> order;
    for (size_t i = 0; i < h->tensors.size(); ++i) {
      TensorInfo &t = h->tensors[i];
      if (batched && t.ptr && t.ptr == cfg.output_tokens) { t.storage = 1; continue; }
      if (batched && meta_in(t.ptr)) { t.storage = 0; continue; }
      if (!t.ptr) { t.storage = next++; continue; }
      order.push_back(i);
    }
    std::sort(order.begin(), order.end(), [&](size_t a, size_t b) {
      return reinterpret_cast<uintptr_t>(h->tensors[a].ptr) < reinterpret_cast<uintptr_t>(h->tensors[b].ptr);
    });
    uintptr_t run_end = 0;
    int run_id = -1;
    for (size_t i : order) {
      TensorInfo &t = h->tensors[i];
      const uintptr_t lo = reinterpret_cast<uintptr_t>(t.ptr), hi = lo + std::max<uint64_t>(t.bytes, 1);
      if (run_id < 0 || lo >= run_end) { run_id = next++; run_end = hi; }
      else run_end = std::max(run_end, hi);
      t.storage = run_id;
    }
  }
  // 4. task graph
  int W = cfg.num_workers > 0 ? std::min(cfg.num_workers, h->num_sms) : h->num_sms;
  GraphInputs in{&h->cfg, &h->tensors, &h->layers, W, 0};
  int rc = build_task_graph(in, &h->graph, &h->error);
  if (rc) return rc;
  CompiledGraph &g = h->graph;
  if (g.num_stages > 8)   // entries 8.. of the 16-entry barrier arrays are scratch (attention stash, accumulator barrier)
    return set_err(h, MPK_ERR_UNSUPPORTED, "internal: more than 8 weight stages planned");
  h->smem_bytes = mpk_kernel_smem_bytes(g.num_stages, g.stage_bytes, g.x_tile_bytes);
  // 5. runtime buffers
  h->counters_bytes = ((uint64_t)g.num_events * 8 + 255) / 256 * 256;
  h->comm_bytes = h->counters_bytes + (uint64_t)2 * g.inbox_floats_per_buffer * 4 + 256;
  rc = dev_alloc(h, (void **)&h->comm, h->comm_bytes); if (rc) return rc;
  rc = dev_alloc(h, (void **)&h->d_status, sizeof(DeviceStatus)); if (rc) return rc;
  rc = dev_alloc(h, (void **)&h->d_request_ids, (uint64_t)cfg.max_num_batched_requests * 4); if (rc) return rc;
  rc = dev_alloc(h, (void **)&h->d_page_queue, (uint64_t)std::max(cfg.max_num_pages, 1) * 4); if (rc) return rc;
  rc = dev_alloc(h, (void **)&h->d_sched, 64); if (rc) return rc;
  rc = dev_alloc(h, (void **)&h->d_attn_scratch, (uint64_t)g.attn_scratch_floats * 4); if (rc) return rc;
  rc = dev_alloc(h, (void **)&h->d_attn_tickets, (uint64_t)std::max<int64_t>(g.attn_tickets, 1) * 4); if (rc) return rc;
  rc = dev_alloc(h, (void **)&h->d_tasks, (uint64_t)g.tasks.size() * sizeof(TaskDesc), false); if (rc) return rc;
  rc = dev_alloc(h, (void **)&h->d_worker_begin, (uint64_t)(W + 1) * 4, false); if (rc) return rc;
  int32_t *snapshot = cfg.paged_kv_indices_snapshot;
  if (!snapshot && !cfg.test_mode && cfg.mode != MPK_MODE_ONLINE_NOTOKEN) {
    rc = dev_alloc(h, (void **)&snapshot, (uint64_t)std::max(cfg.max_num_pages, 1) * 4); if (rc) return rc;
  }
  rc = upload_tensor_maps(h); if (rc) return rc;
  if (!dry) {
    CU(cudaMemcpy(h->d_tasks, g.tasks.data(), g.tasks.size() * sizeof(TaskDesc), cudaMemcpyHostToDevice));
    CU(cudaMemcpy(h->d_worker_begin, g.worker_begin.data(), (W + 1) * 4, cudaMemcpyHostToDevice));
  }
  KernelParams &P = h->params;
  std::memset(&P, 0, sizeof(P));
  P.tasks = h->d_tasks;
  P.worker_begin = h->d_worker_begin;
  P.counters = reinterpret_cast<unsigned long long *>(h->comm);
  P.status = h->d_status;
  h->peer_comm[cfg.rank] = h->comm;
  for (int r = 0; r < kMaxWorld; ++r) { P.peer_counters[r] = nullptr; P.peer_inbox[r] = nullptr; }
  P.peer_counters[cfg.rank] = P.counters;
  P.peer_inbox[cfg.rank] = reinterpret_cast<float *>(h->comm + h->counters_bytes);
  P.meta.step = cfg.step; P.meta.tokens = cfg.tokens; P.meta.input_tokens = cfg.input_tokens;
  P.meta.output_tokens = cfg.output_tokens; P.meta.prompt_lengths = cfg.prompt_lengths;
  P.meta.qo_indptr = cfg.qo_indptr; P.meta.paged_kv_indptr = cfg.paged_kv_indptr;
  P.meta.paged_kv_indices = cfg.paged_kv_indices; P.meta.paged_kv_last_page_len = cfg.paged_kv_last_page_len;
  P.meta.paged_kv_indices_snapshot = snapshot;
  P.meta.request_ids = h->d_request_ids; P.meta.page_queue = h->d_page_queue; P.meta.sched_scalars = h->d_sched;
  P.attn_scratch = h->d_attn_scratch;
  P.attn_tickets = h->d_attn_tickets;
  P.profiler = cfg.profiler_buffer;
  P.profiler_entries = cfg.profiler_entries;
  P.eos_token_id = cfg.eos_token_id;
  P.num_workers = W;
  P.test_mode = cfg.test_mode;
  P.world_size = cfg.world_size;
  P.rank = cfg.rank;
  P.max_seq_length = cfg.max_seq_length;
  P.max_num_batched_requests = cfg.max_num_batched_requests;
  P.max_num_batched_tokens = cfg.max_num_batched_tokens;
  P.max_num_pages = cfg.max_num_pages;
  P.page_size = cfg.page_size;
  P.total_num_requests = cfg.total_num_requests;
  P.num_stages = g.num_stages;
  P.stage_bytes = g.stage_bytes;
  P.x_tile_bytes = g.x_tile_bytes;
  P.max_inflight = g.num_stages;
  P.general_kernel = g.general_kernel ? 1 : 0;
  P.tmaps = h->d_tmaps;
  P.use_tmem = g.use_tmem ? 1 : 0;
  P.tc_tokens = g.tc_tokens;
  P.meta_static = (cfg.test_mode || cfg.mode == MPK_MODE_ONLINE_NOTOKEN) ? 1 : 0;
  P.ll_row_words = 0;
  P.ll_buffer_words = (int32_t)g.inbox_floats_per_buffer;
  for (const TaskDesc &t : g.tasks)
    if (t.type == TASK_LINEAR && t.a[L_EPI] == EPI_PUSH_LL) {
      if (P.ll_row_words == 0) P.ll_row_words = t.a[L_N];
      else if (P.ll_row_words != t.a[L_N]) { P.ll_row_words = 0; break; }
    }
  P.tp_extensions = 0;
  for (const TaskDesc &t : g.tasks) if (t.type == TASK_ARGMAX_EXCHANGE) P.tp_extensions = 1;
  P.quiet_streaming = 0;
  P.kv_l2_prefetch = 1;
  P.spin_limit = 4000;   // milliseconds a launch may wait before it gives up
  if (const char *e = getenv("MPK_SPIN_LIMIT_MS")) P.spin_limit = (uint32_t)std::max(1, std::min(atoi(e), 60000));
  if (!dry) {
    int e = mpk_kernel_prepare(h->smem_bytes);
    if (e) return set_err(h, MPK_ERR_CUDA, std::string("cudaFuncSetAttribute(smem=") + std::to_string(h->smem_bytes) +
                                               "): " + cudaGetErrorString((cudaError_t)e));
  }
  h->compiled = true;
  h->needs_reset = true;
  return MPK_OK;
}

int mpk_comm_export(mpk_handle *h, void *ipc_handle_64B) {
  if (!h || !ipc_handle_64B) return MPK_ERR_INVALID;
  if (!h->compiled) return set_err(h, MPK_ERR_STATE, "comm_export before compile");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (h->cfg.dry_run) { std::memset(ipc_handle_64B, 0, 64); return MPK_OK; }
  CU(cudaSetDevice(h->cfg.device));
  cudaIpcMemHandle_t hd;
  CU(cudaIpcGetMemHandle(&hd, h->comm));
  std::memcpy(ipc_handle_64B, &hd, 64);
  return MPK_OK;
}

static int link_peer(mpk_handle *h, int peer_rank, void *base) {
  h->peer_comm[peer_rank] = base;
  h->params.peer_counters[peer_rank] = reinterpret_cast<unsigned long long *>(base);
  h->params.peer_inbox[peer_rank] = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(base) + h->counters_bytes);
  return MPK_OK;
}

int mpk_comm_import(mpk_handle *h, int peer_rank, const void *ipc_handle_64B) {
  if (!h || !ipc_handle_64B) return MPK_ERR_INVALID;
  if (!h->compiled) return set_err(h, MPK_ERR_STATE, "comm_import before compile");
  if (peer_rank < 0 || peer_rank >= h->cfg.world_size) return set_err(h, MPK_ERR_INVALID, "bad peer rank");
  if (peer_rank == h->cfg.rank || h->cfg.dry_run) return MPK_OK;
  CU(cudaSetDevice(h->cfg.device));
  cudaIpcMemHandle_t hd;
  std::memcpy(&hd, ipc_handle_64B, 64);
  void *base = nullptr;
  CU(cudaIpcOpenMemHandle(&base, hd, cudaIpcMemLazyEnablePeerAccess));
  h->peer_opened[peer_rank] = true;
  return link_peer(h, peer_rank, base);
}

int mpk_comm_link_local(mpk_handle *h, int peer_rank, mpk_handle *peer) {
  if (!h || !peer) return MPK_ERR_INVALID;
  if (!h->compiled || !peer->compiled) return set_err(h, MPK_ERR_STATE, "comm_link_local before compile");
  if (peer_rank < 0 || peer_rank >= h->cfg.world_size) return set_err(h, MPK_ERR_INVALID, "bad peer rank");
  if (peer_rank == h->cfg.rank) return MPK_OK;
  if (!h->cfg.dry_run && h->cfg.device != peer->cfg.device) {
    CU(cudaSetDevice(h->cfg.device));
    cudaError_t e = cudaDeviceEnablePeerAccess(peer->cfg.device, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
      return set_err(h, MPK_ERR_CUDA, std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e));
    cudaGetLastError();
  }
  return link_peer(h, peer_rank, peer->comm);
}

int mpk_reset(mpk_handle *h, void *cuda_stream) {
  if (!h) return MPK_ERR_INVALID;
  if (!h->compiled) return set_err(h, MPK_ERR_STATE, "reset before compile");
  if (h->cfg.dry_run) { h->needs_reset = false; return MPK_OK; }
  const mpk_config &cfg = h->cfg;
  cudaStream_t st = (cudaStream_t)cuda_stream;
  CU(cudaSetDevice(cfg.device));
  CU(cudaMemsetAsync(h->comm, 0, h->comm_bytes, st));   // event counters and both inbox buffers
  CU(cudaMemsetAsync(h->d_status, 0, sizeof(DeviceStatus), st));
  CU(cudaMemsetAsync(h->d_attn_tickets, 0, (size_t)std::max<int64_t>(h->graph.attn_tickets, 1) * 4, st));
  if (!cfg.test_mode && cfg.mode != MPK_MODE_ONLINE_NOTOKEN) {
    // init_kernel, include/mirage/persistent_kernel/persistent_kernel.cuh:149-166 (offline only: in online_notoken
    // the batch description belongs to the caller and is left alone)
    CU(cudaMemsetAsync(cfg.step, 0, (size_t)cfg.total_num_requests * 4, st));
    CU(cudaMemsetAsync(h->d_request_ids, 0xff, (size_t)cfg.max_num_batched_requests * 4, st));
    CU(cudaMemsetAsync(cfg.qo_indptr, 0, (size_t)(cfg.max_num_batched_requests + 1) * 4, st));
    CU(cudaMemsetAsync(cfg.paged_kv_indptr, 0, (size_t)(cfg.max_num_batched_requests + 1) * 4, st));
    std::vector<int32_t> ring(cfg.max_num_pages);
    for (int i = 0; i < cfg.max_num_pages; ++i) ring[i] = i;
    CU(cudaMemcpyAsync(h->d_page_queue, ring.data(), ring.size() * 4, cudaMemcpyHostToDevice, st));
    const int32_t sc[3] = {0, cfg.max_num_pages, 0};
    CU(cudaMemcpyAsync(h->d_sched, sc, sizeof(sc), cudaMemcpyHostToDevice, st));
    CU(cudaStreamSynchronize(st));   // the host staging buffers above go out of scope
  }
  h->needs_reset = false;
  h->reset_after_error = false;
  return MPK_OK;
}

int mpk_launch(mpk_handle *h, void *cuda_stream, int num_steps) {
  if (!h) return MPK_ERR_INVALID;
  if (!h->compiled) return set_err(h, MPK_ERR_STATE, "launch before compile");
  if (h->cfg.dry_run) return set_err(h, MPK_ERR_STATE, "dry-run handles cannot launch");
  for (int r = 0; r < h->cfg.world_size; ++r)
    if (!h->params.peer_inbox[r]) return set_err(h, MPK_ERR_STATE, "peer " + std::to_string(r) + " not linked");
  if (h->needs_reset) {
    // After a device wait expired the counters and inboxes must be cleared before the next launch.  With one rank
    // that is done here; with several ranks the clearing is a collective (no rank may push before every rank has
    // cleared, see mpk_reset in the header) that only the caller can fence, so the launch is refused instead.
    if (h->reset_after_error && h->cfg.world_size > 1)
      return set_err(h, MPK_ERR_STATE, "a device wait timed out: call mpk_reset on every rank (collectively) before launching again");
    int rc = mpk_reset(h, cuda_stream);
    if (rc) return rc;
  }
  CU(cudaSetDevice(h->cfg.device));
  for (int i = 0; i < num_steps; ++i) {
    int e = mpk_kernel_launch(&h->params, h->smem_bytes, cuda_stream);
    if (e) return set_err(h, MPK_ERR_CUDA, std::string("megakernel launch: ") + cudaGetErrorString((cudaError_t)e));
  }
  return MPK_OK;
}

int mpk_sync_status(mpk_handle *h, void *cuda_stream, mpk_status *out) {
  if (!h || !out) return MPK_ERR_INVALID;
  if (!h->compiled) return set_err(h, MPK_ERR_STATE, "status before compile");
  std::memset(out, 0, sizeof(*out));
  if (h->cfg.dry_run) return MPK_OK;
  CU(cudaSetDevice(h->cfg.device));
  CU(cudaStreamSynchronize((cudaStream_t)cuda_stream));
  DeviceStatus st;
  CU(cudaMemcpy(&st, h->d_status, sizeof(st), cudaMemcpyDeviceToHost));
  out->error = st.error; out->where = st.where; out->worker = st.worker; out->task = st.task;
  out->all_done = st.all_done; out->active_tokens = st.active_tokens; out->iteration = st.iteration;
  if (getenv("MPK_PRINT_KERNEL_TIMES")) {
    for (int i = 0; i < 8; ++i) {
      const int a = (int)((st.iteration + 1 + i) & 7), b = (int)((st.iteration + 2 + i) & 7);
      fprintf(stderr, "[mpk] it%%8=%d kernel %.1f us, gap to next %.1f us\n", a, (st.t_end[a] - st.t_start[a]) / 1e3,
              i < 7 ? ((double)st.t_start[b] - (double)st.t_end[a]) / 1e3 : 0.0);
    }
  }
  if (st.error != 0) {
    h->needs_reset = true;
    h->reset_after_error = true;
    return set_err(h, MPK_ERR_TIMEOUT, "device wait timed out (where=" + std::to_string(st.where) + ", worker=" +
                                           std::to_string(st.worker) + ", task=" + std::to_string(st.task) + ")");
  }
  return MPK_OK;
}

int mpk_tensor_ptr(mpk_handle *h, int tensor_id, void **device_ptr, uint64_t *bytes) {
  if (!h || tensor_id < 0 || tensor_id >= (int)h->tensors.size()) return set_err(h, MPK_ERR_INVALID, "bad tensor id");
  if (device_ptr) *device_ptr = h->tensors[tensor_id].ptr;
  if (bytes) *bytes = h->tensors[tensor_id].bytes;
  return MPK_OK;
}

int mpk_graph_info(mpk_handle *h, int *num_tasks, int *num_events, int *num_workers, int *num_layers_folded) {
  if (!h || !h->compiled) return set_err(h, MPK_ERR_STATE, "graph_info before compile");
  if (num_tasks) *num_tasks = (int)h->graph.tasks.size();
  if (num_events) *num_events = h->graph.num_events;
  if (num_workers) *num_workers = h->graph.num_workers;
  if (num_layers_folded) *num_layers_folded = h->graph.num_folded;
  return MPK_OK;
}

int64_t mpk_dump_task_graph(mpk_handle *h, char *buf, int64_t buf_bytes) {
  if (!h || !h->compiled) return MPK_ERR_STATE;
  const std::string s = dump_task_graph(h->graph, h->tensors, h->layers);
  if (buf && buf_bytes > 0) {
    const int64_t n = std::min<int64_t>(buf_bytes - 1, (int64_t)s.size());
    std::memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return (int64_t)s.size() + 1;
}

int64_t mpk_weight_bytes_per_step(mpk_handle *h) {
  if (!h || !h->compiled) return MPK_ERR_STATE;
  return h->graph.weight_bytes;
}

}  // extern "C"
