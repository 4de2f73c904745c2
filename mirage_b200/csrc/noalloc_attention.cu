// mpk_paged_decode_attention_noalloc: split-KV paged GQA decode attention as a stand-alone launch whose
// scratch memory is a fixed array inside the library image.
//
// Who needs this: callers that are not allowed to allocate device memory when they call into the library --
// code running while a CUDA graph is being captured, a serving loop whose memory pool owns every byte of the
// device and forbids cudaMalloc after start-up, or a plugin host that only hands the library a stream.  The
// handle-based path (mpk_compile) allocates its split-KV scratch with cudaMalloc; this entry point never calls
// cudaMalloc, cudaFree or any other allocating routine.
//
// The scratch (per-chunk softmax partials and the per-(request, kv head) arrival tickets) lives in the
// file-scope array `g_noalloc_scratch` below: kNoAllocScratchBytes (4 MiB) of every GPU that loads the library,
// held until the process exits.  Problem sizes that do not fit are rejected with an error, not truncated.
//
// Rules for callers:
//   * The first call on a device looks up the device address of the array (cudaGetSymbolAddress).  Make that
//     first call outside of any stream capture.
//   * All calls share the one array.  Two calls whose kernels may overlap on the GPU (different streams, or
//     different host threads on the same device) race on it; serialise them on one stream.
//   * The array keeps the previous call's contents.  The only part that must start at zero, the tickets, is
//     cleared on the caller's stream before every launch.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/mpk_b200.h"

namespace {

constexpr size_t kNoAllocScratchBytes = 4u << 20;
constexpr int kMaxTickets = 4096;                       // request x kv-head pairs
constexpr size_t kTicketBytes = kMaxTickets * sizeof(unsigned int);
constexpr int kPartialFloats = 2 + 128;                 // running max, running sum, 128 output dims
constexpr int kMaxDevices = 64;

// Device code may name this array directly; host code must not pass the symbol itself to a kernel (on the host
// it is only a stand-in) and uses the address cudaGetSymbolAddress returns.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

__device__ __forceinline__ float lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct Args {
  const __nv_bfloat16 *qkv;       // [requests, ld_qkv]; per kv head [q x G | k | v] of 128 each
  __nv_bfloat16 *k_cache, *v_cache;   // [pages, page_size, kv_heads, 128]
  __nv_bfloat16 *out;             // [requests, ld_out]
  const int32_t *kv_indptr, *kv_indices, *kv_last_page_len;
  unsigned int *tickets;          // scratch: [requests * kv_heads]
  float *partials;                // scratch: [requests][q heads][chunks][130]
  int num_q_heads, num_kv_heads, page_size, ld_qkv, ld_out, num_chunks;
};

// grid (chunks, kv heads, requests), 128 threads.  Warp w walks positions start + w, start + w + 4, ...; lane l
// owns dims 4l..4l+3.  The block that owns position seq_len-1 appends the new K/V row first.
template <int G>
__global__ void __launch_bounds__(128) noalloc_decode_attention(const Args a) {
  const int chunk = blockIdx.x, head = blockIdx.y, req = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kv0 = a.kv_indptr[req];
  const int npages = a.kv_indptr[req + 1] - kv0;
  // An empty sequence (no page, or a length that works out to <= 0) has nothing to attend to: it skips the append
  // and the loop, still takes its ticket, and the merging block writes zeros.
  const int seq_len = max((npages - 1) * a.page_size + a.kv_last_page_len[req], 0);
  int L = (seq_len + a.num_chunks - 1) / a.num_chunks;
  L = max((L + 15) & ~15, 16);
  const int n_active = (seq_len + L - 1) / L;
  const int start = chunk * L, end = min(seq_len, start + L);
  const int hq = a.num_q_heads;
  const __nv_bfloat16 *row = a.qkv + (size_t)req * a.ld_qkv + (size_t)head * (G + 2) * 128;
  auto kv_off = [&](int pos) {
    const int pi = pos / a.page_size;
    const int pid = a.kv_indices[kv0 + pi];
    return (((size_t)pid * a.page_size + (pos - pi * a.page_size)) * a.num_kv_heads + head) * 128;
  };
  if (seq_len - 1 >= start && seq_len - 1 < end && warp == 0) {
    const size_t off = kv_off(seq_len - 1) + lane * 4;
    *reinterpret_cast<uint2 *>(a.k_cache + off) = *reinterpret_cast<const uint2 *>(row + G * 128 + lane * 4);
    *reinterpret_cast<uint2 *>(a.v_cache + off) = *reinterpret_cast<const uint2 *>(row + (G + 1) * 128 + lane * 4);
  }
  __syncthreads();
  const float qscale = 0.08838834764831845f * 1.4426950408889634f;   // 1/sqrt(128) * log2(e)
  float q[G][4], m[G], l[G], o[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint2 r = *reinterpret_cast<const uint2 *>(row + g * 128 + lane * 4);
    q[g][0] = lo(r.x) * qscale; q[g][1] = hi(r.x) * qscale; q[g][2] = lo(r.y) * qscale; q[g][3] = hi(r.y) * qscale;
    m[g] = -INFINITY; l[g] = 0.f;
    o[g][0] = o[g][1] = o[g][2] = o[g][3] = 0.f;
  }
  for (int pos = start + warp; pos < end; pos += 4) {
    const size_t off = kv_off(pos) + lane * 4;
    const uint2 kr = *reinterpret_cast<const uint2 *>(a.k_cache + off);
    const uint2 vr = *reinterpret_cast<const uint2 *>(a.v_cache + off);
    const float kf[4] = {lo(kr.x), hi(kr.x), lo(kr.y), hi(kr.y)};
    const float vf[4] = {lo(vr.x), hi(vr.x), lo(vr.y), hi(vr.y)};
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float s = wsum(q[g][0] * kf[0] + q[g][1] * kf[1] + q[g][2] * kf[2] + q[g][3] * kf[3]);
      const float mn = fmaxf(m[g], s);
      const float corr = exp2f(m[g] - mn), p = exp2f(s - mn);
      m[g] = mn;
      l[g] = l[g] * corr + p;
#pragma unroll
      for (int i = 0; i < 4; ++i) o[g][i] = o[g][i] * corr + p * vf[i];
    }
  }
  __shared__ float s_m[4][G], s_l[4][G], s_o[4][G][128];
  __shared__ int s_last;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
#pragma unroll
    for (int i = 0; i < 4; ++i) s_o[warp][g][lane * 4 + i] = o[g][i];
  }
  __syncthreads();
  for (int idx = tid; idx < G * 128; idx += 128) {
    const int g = idx >> 7, d = idx & 127;
    float M = -INFINITY;
    for (int w = 0; w < 4; ++w) M = fmaxf(M, s_m[w][g]);
    float Ls = 0.f, O = 0.f;
    for (int w = 0; w < 4; ++w) {
      const float sc = (s_m[w][g] == -INFINITY) ? 0.f : exp2f(s_m[w][g] - M);
      Ls += s_l[w][g] * sc;
      O += s_o[w][g][d] * sc;
    }
    float *p = a.partials + (((size_t)req * hq + head * G + g) * a.num_chunks + chunk) * kPartialFloats;
    p[2 + d] = O;
    if (d == 0) { p[0] = M; p[1] = Ls; }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned int old = atomicAdd(&a.tickets[req * a.num_kv_heads + head], 1u);
    s_last = (old + 1u == (unsigned)a.num_chunks) ? 1 : 0;
    __threadfence();
  }
  __syncthreads();
  if (!s_last) return;
  for (int idx = tid; idx < G * 128; idx += 128) {
    const int g = idx >> 7, d = idx & 127;
    const float *p = a.partials + ((size_t)req * hq + head * G + g) * a.num_chunks * kPartialFloats;
    float M = -INFINITY;
    for (int c = 0; c < n_active; ++c) M = fmaxf(M, __ldcg(&p[(size_t)c * kPartialFloats]));
    float Ls = 0.f, O = 0.f;
    for (int c = 0; c < n_active; ++c) {
      const float mc = __ldcg(&p[(size_t)c * kPartialFloats]);
      const float sc = (mc == -INFINITY) ? 0.f : exp2f(mc - M);
      Ls += __ldcg(&p[(size_t)c * kPartialFloats + 1]) * sc;
      O += __ldcg(&p[(size_t)c * kPartialFloats + 2 + d]) * sc;
    }
    a.out[(size_t)req * a.ld_out + (size_t)(head * G + g) * 128 + d] = __float2bfloat16_rn(Ls > 0.f ? O / Ls : 0.f);
  }
}

std::mutex g_setup_mutex;
void *g_scratch_addr[kMaxDevices] = {};

int fail(char *err, size_t err_len, int code, const char *fmt, long long a = 0, long long b = 0) {
  if (err && err_len) snprintf(err, err_len, fmt, a, b);
  return code;
}

}  // namespace

extern "C" int mpk_paged_decode_attention_noalloc(const void *qkv, void *k_cache, void *v_cache, void *out,
                                                  const int32_t *kv_indptr, const int32_t *kv_indices,
                                                  const int32_t *kv_last_page_len, int num_requests, int num_q_heads,
                                                  int num_kv_heads, int page_size, int64_t ld_qkv, int64_t ld_out,
                                                  int num_chunks, void *cuda_stream, char *err, size_t err_len) {
  if (!qkv || !k_cache || !v_cache || !out || !kv_indptr || !kv_indices || !kv_last_page_len)
    return fail(err, err_len, MPK_ERR_INVALID, "mpk_paged_decode_attention_noalloc: null pointer argument");
  if (num_requests < 1 || num_kv_heads < 1 || num_q_heads < 1 || page_size < 1 || num_chunks < 1 ||
      num_q_heads % num_kv_heads != 0)
    return fail(err, err_len, MPK_ERR_INVALID, "mpk_paged_decode_attention_noalloc: bad sizes");
  const int G = num_q_heads / num_kv_heads;
  if (G != 1 && G != 2 && G != 4 && G != 8)
    return fail(err, err_len, MPK_ERR_UNSUPPORTED, "GQA group size %lld not supported (1, 2, 4, 8)", G);
  // The kernel reads [q x G | k | v] rows of 128 bf16 per kv head as 8-byte vectors: the rows must be wide enough,
  // and the strides and base addresses 8-byte aligned (a misaligned vector load faults the context).
  const long long qkv_width = (long long)num_kv_heads * (G + 2) * 128, out_width = (long long)num_q_heads * 128;
  if (ld_qkv < qkv_width || ld_out < out_width || ld_qkv > 0x7fffffffll || ld_out > 0x7fffffffll)
    return fail(err, err_len, MPK_ERR_INVALID, "row strides (%lld, %lld elements) are narrower than the packed q|k|v / output rows", ld_qkv,
                ld_out);
  if (ld_qkv % 4 != 0 || ld_out % 4 != 0)
    return fail(err, err_len, MPK_ERR_INVALID, "row strides (%lld, %lld elements) must be multiples of 4", ld_qkv, ld_out);
  if (((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 7u)
    return fail(err, err_len, MPK_ERR_INVALID, "qkv, k_cache, v_cache and out must be 8-byte aligned");
  if (((uintptr_t)kv_indptr | (uintptr_t)kv_indices | (uintptr_t)kv_last_page_len) & 3u)
    return fail(err, err_len, MPK_ERR_INVALID, "the kv index arrays must be 4-byte aligned");
  const long long tickets = (long long)num_requests * num_kv_heads;
  if (tickets > kMaxTickets)
    return fail(err, err_len, MPK_ERR_UNSUPPORTED,
                "requests x kv_heads = %lld exceeds the %lld tickets of the built-in scratch", tickets, kMaxTickets);
  const long long need = (long long)kTicketBytes +
                         (long long)num_requests * num_q_heads * num_chunks * kPartialFloats * (long long)sizeof(float);
  if (need > (long long)kNoAllocScratchBytes)
    return fail(err, err_len, MPK_ERR_UNSUPPORTED,
                "problem needs %lld bytes of scratch; the built-in scratch holds %lld (use fewer chunks or requests)",
                need, (long long)kNoAllocScratchBytes);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(err, err_len, MPK_ERR_CUDA, "cudaGetDevice failed or device ordinal out of range (%lld)", dev);
  void *scratch = nullptr;
  {
    // once per device, with that device current: resolve the device address of the scratch array
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[dev]) {
      void *p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || !p)
        return fail(err, err_len, MPK_ERR_CUDA, "cudaGetSymbolAddress(g_noalloc_scratch) failed: code %lld", (int)e);
      g_scratch_addr[dev] = p;
    }
    scratch = g_scratch_addr[dev];
  }
  cudaStream_t st = (cudaStream_t)cuda_stream;
  e = cudaMemsetAsync(scratch, 0, (size_t)tickets * sizeof(unsigned int), st);   // tickets must start at zero
  if (e != cudaSuccess) return fail(err, err_len, MPK_ERR_CUDA, "cudaMemsetAsync(tickets) failed: code %lld", (int)e);
  Args a;
  a.qkv = (const __nv_bfloat16 *)qkv;
  a.k_cache = (__nv_bfloat16 *)k_cache;
  a.v_cache = (__nv_bfloat16 *)v_cache;
  a.out = (__nv_bfloat16 *)out;
  a.kv_indptr = kv_indptr; a.kv_indices = kv_indices; a.kv_last_page_len = kv_last_page_len;
  a.tickets = (unsigned int *)scratch;
  a.partials = (float *)((unsigned char *)scratch + kTicketBytes);
  a.num_q_heads = num_q_heads; a.num_kv_heads = num_kv_heads; a.page_size = page_size;
  a.ld_qkv = (int)ld_qkv; a.ld_out = (int)ld_out; a.num_chunks = num_chunks;
  const dim3 grid(num_chunks, num_kv_heads, num_requests);
  switch (G) {
    case 1: noalloc_decode_attention<1><<<grid, 128, 0, st>>>(a); break;
    case 2: noalloc_decode_attention<2><<<grid, 128, 0, st>>>(a); break;
    case 4: noalloc_decode_attention<4><<<grid, 128, 0, st>>>(a); break;
    default: noalloc_decode_attention<8><<<grid, 128, 0, st>>>(a); break;
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(err, err_len, MPK_ERR_CUDA, "kernel launch failed: code %lld", (int)e);
  return MPK_OK;
}
