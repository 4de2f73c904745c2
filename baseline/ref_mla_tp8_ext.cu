// Host wrapper (this repo's own code) around the reference's absorbed-MLA decode kernel for 16 local heads,
// `kernel::mla_mtp_tp8::mla_mtp_tp8_main` / `mla_mtp_tp8_reduce`
// (include/mirage/persistent_kernel/tasks/blackwell/mla_mtp_decode_tp8_sm100.cuh, included from the reference checkout
// at build time, unmodified).  The reference's own stand-alone driver for these functions
// (tests/runtime_python/blackwell/sm100_mla_mtp_decode/test_tp8_wrapper.cu) sizes its query and output buffers for one
// request whatever --b says, so it cannot be used for a batch; this wrapper launches the same two device functions on
// the same grids with buffers sized for `requests`, taking torch tensors.
//
//   init(Q [requests, q_len_padded, 16, 576] bf16, KV [requests, kv_len, 576] bf16, q_len_real, softmax_scale)
//   run(O [requests, q_len_padded, 16, 512] bf16)        -- asynchronous: main + reduce on the current stream 0
#include "mirage/persistent_kernel/tasks/blackwell/mla_mtp_decode_tp8_sm100.cuh"

#include <torch/extension.h>

using namespace kernel::mla_mtp_tp8;

template <bool SINGLE_TILE>
__global__ __launch_bounds__(TB) void main_shim(const __grid_constant__ CUtensorMap q_map,
                                                const __grid_constant__ CUtensorMap kv_map, nv_bfloat16 *o_acc,
                                                float *lse, float scale, int kv_len, int splits, int q_len, int qpg,
                                                int q_len_real) {
  mla_mtp_tp8_main<SINGLE_TILE>(&q_map, &kv_map, o_acc, lse, scale, kv_len, splits, q_len, qpg, q_len_real, blockIdx.x,
                                blockIdx.y);
}

__global__ __launch_bounds__(RD_TB, 4) void reduce_shim(nv_bfloat16 const *o_acc, float const *lse, nv_bfloat16 *out,
                                                        int splits, int groups, int q_len, int qpg) {
  mla_mtp_tp8_reduce(o_acc, lse, out, splits, groups, q_len, qpg, blockIdx.x, blockIdx.y, blockIdx.z);
}

namespace {
struct State {
  CUtensorMap q_map, kv_map;
  torch::Tensor o_acc, lse, q, kv;
  int requests = 0, kv_len = 0, q_len = 0, q_len_real = 0, splits = 0, groups = 0;
  float scale = 0.f;
  bool ready = false;
} S;
constexpr int kQueriesPerGroup = 2;

void encode(CUtensorMap *map, void *base, uint64_t rows, uint32_t box_rows) {
  // [rows, 576] bf16 seen as 9 slabs of 64 columns: {64 columns, rows, 9 slabs}, 128-byte swizzle
  uint64_t dims[3] = {64, rows, (uint64_t)K_ITERS};
  uint64_t strides[2] = {(uint64_t)D_K * 2, 128};
  uint32_t box[3] = {64, box_rows, 1};
  uint32_t elem[3] = {1, 1, 1};
  CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, elem,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed: ", (int)r);
}
}  // namespace

void init(torch::Tensor q, torch::Tensor kv, int64_t q_len_real, double scale) {
  TORCH_CHECK(q.is_cuda() && kv.is_cuda() && q.is_contiguous() && kv.is_contiguous());
  TORCH_CHECK(q.scalar_type() == torch::kBFloat16 && kv.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(q.dim() == 4 && q.size(2) == NUM_HEADS && q.size(3) == D_K, "Q must be [requests, q_len, 16, 576]");
  TORCH_CHECK(kv.dim() == 3 && kv.size(0) == q.size(0) && kv.size(2) == D_K, "KV must be [requests, kv_len, 576]");
  TORCH_CHECK(q.size(1) % kQueriesPerGroup == 0 && q_len_real >= 1 && q_len_real <= q.size(1) && q.size(1) <= 8);
  S.requests = (int)q.size(0);
  S.q_len = (int)q.size(1);
  S.q_len_real = (int)q_len_real;
  S.kv_len = (int)kv.size(1);
  S.groups = S.q_len / kQueriesPerGroup;
  S.splits = (S.kv_len + TILE_S - 1) / TILE_S;       // one 128-row tile per split, as the reference's driver chooses
  S.scale = (float)scale;
  S.q = q;
  S.kv = kv;
  const int64_t blocks = (int64_t)S.requests * S.groups * S.splits;
  TORCH_CHECK(blocks * D_V * 128 < (int64_t)1 << 31, "partial buffer index would overflow the kernel's int arithmetic");
  S.o_acc = torch::zeros({blocks * D_V * 128}, torch::dtype(torch::kBFloat16).device(q.device()));
  S.lse = torch::zeros({blocks * 128}, torch::dtype(torch::kFloat32).device(q.device()));
  encode(&S.q_map, q.data_ptr(), (uint64_t)S.requests * S.q_len * NUM_HEADS, NUM_HEADS);
  encode(&S.kv_map, kv.data_ptr(), (uint64_t)S.requests * S.kv_len, TILE_S);
  cudaFuncSetAttribute(main_shim<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_SIZE);
  S.ready = true;
}

void run(torch::Tensor out) {
  TORCH_CHECK(S.ready, "init first");
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == torch::kBFloat16 &&
              out.numel() == (int64_t)S.requests * S.q_len * NUM_HEADS * D_V);
  dim3 grid(S.groups * S.splits, S.requests);
  main_shim<true><<<grid, TB, SMEM_SIZE>>>(S.q_map, S.kv_map, (nv_bfloat16 *)S.o_acc.data_ptr(),
                                           (float *)S.lse.data_ptr(), S.scale, S.kv_len, S.splits, S.q_len,
                                           kQueriesPerGroup, S.q_len_real);
  dim3 rgrid((D_V + RD_DV - 1) / RD_DV, S.groups, S.requests);
  reduce_shim<<<rgrid, RD_TB>>>((nv_bfloat16 const *)S.o_acc.data_ptr(), (float const *)S.lse.data_ptr(),
                                (nv_bfloat16 *)out.data_ptr(), S.splits, S.groups, S.q_len, kQueriesPerGroup);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("init", &init, "tensor maps + partial buffers");
  m.def("run", &run, "launch decode + merge (asynchronous)");
}
