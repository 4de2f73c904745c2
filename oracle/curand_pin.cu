// TEST INFRASTRUCTURE ONLY: runs NVIDIA's own cuRAND device generator (the third-party dependency the reference's
// sampling task calls, tasks/common/sampling.cuh:100-152) so that oracle/sampling_ops.py, a restatement of
// Philox4x32-10 and of the uniform -> Gumbel transform, can be pinned against it on a GPU.  Built by
// oracle/build_ref.py into oracle/_ref/libcurand_pin.so with -use_fast_math, the flag the reference compiles its
// kernel with (python/mirage/mpk/persistent_kernel.py:253).  Nothing in the product links or loads this file.
#include <cuda_runtime.h>
#include <curand_kernel.h>
#include <stdint.h>

namespace {
__global__ void pin_kernel(unsigned long long seed, unsigned long long first_subsequence, int groups, float *uniform,
                           float *gumbel) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  curandStatePhilox4_32_10_t state;
  curand_init(seed, first_subsequence + 4ull * (unsigned long long)g, 0ull, &state);
  const float4 u = curand_uniform4(&state);
  const float us[4] = {u.x, u.y, u.z, u.w};
  for (int e = 0; e < 4; ++e) {
    uniform[g * 4 + e] = us[e];
    gumbel[g * 4 + e] = -0.6931471806f * log2f(-log2f(us[e] + 1e-20f) + 1e-20f);
  }
}
}  // namespace

// uniform / gumbel: DEVICE pointers to 4 * groups floats.  Returns the cudaError_t of the launch + synchronise.
extern "C" int curand_pin_fill(unsigned long long seed, unsigned long long first_subsequence, int groups, float *uniform,
                               float *gumbel) {
  pin_kernel<<<(groups + 255) / 256, 256>>>(seed, first_subsequence, groups, uniform, gumbel);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  return (int)e;
}
