// The decode megakernel: one launch executes one iteration of the task graph.
//
// Replaces the reference's persistent runtime (worker/scheduler loops and queues,
// include/mirage/persistent_kernel/persistent_kernel.cuh:513-1082) and the task bodies
// it dispatches to (include/mirage/persistent_kernel/tasks/**) for the decode path.
//
// Structure of a worker CTA (one per SM, 288 threads):
//   * warp 8 is the weight streamer.  It walks the worker's task list ahead of the
//     compute warps and issues cp.async.bulk copies of the weight rows every linear
//     task will need into a ring of 32 KB shared-memory stages guarded by mbarriers.
//     Weights never depend on events, so the stream keeps HBM busy across task
//     boundaries, dependency waits and attention tasks.
//   * warps 0-7 execute tasks in order: acquire-poll the task's event counters, run
//     the body, release-increment the trigger counter.
// Counters grow monotonically: a dependency is complete when
// counter >= arrivals_per_iteration * iteration.  The iteration number lives in device
// memory and is advanced by the last CTA to leave the kernel, so a captured CUDA graph
// of launches can be replayed.
//
// Every wait (event counter, mbarrier) is bounded by a wall-clock budget; on expiry the
// CTA records where it gave up, raises a global abort flag that all other waits poll,
// drains its own in-flight copies and returns.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "device_utils.cuh"
#include "runtime_types.h"

namespace mpk {

struct Smem {
  uint8_t *stages;      // num_stages * stage_bytes
  uint8_t *xtile;       // x_tile_bytes (activation tile / attention scratch)
  float *partial;       // kPartialBytes (directly after xtile)
  uint64_t *full;       // [num_stages]
  uint64_t *empty;      // [num_stages]
  TaskDesc *desc;       // [2]
  float *red;           // [64]
  int *flags;           // [0] abort  [1] broadcast scratch
  uint64_t *acc_bar;    // tcgen05 path: "accumulators complete / activation tile free" barrier (count 1)
  uint32_t *tmem_holder;   // tensor-memory base address written by tcgen05.alloc
};

constexpr int kMiscBytes = 1536;
constexpr int kStashRing = 16;     // attention stash records of the general instantiation (32 bytes each, after the flags)

__device__ __forceinline__ Smem carve(uint8_t *base, const KernelParams &P) {
  Smem s;
  s.stages = base;
  s.xtile = base + (size_t)P.num_stages * P.stage_bytes;
  s.partial = reinterpret_cast<float *>(s.xtile + P.x_tile_bytes);
  uint8_t *misc = reinterpret_cast<uint8_t *>(s.partial) + kPartialBytes;
  s.full = reinterpret_cast<uint64_t *>(misc);            // 16 * 8
  s.empty = s.full + 16;                                    // 16 * 8
  s.desc = reinterpret_cast<TaskDesc *>(misc + 256);        // 2 * 224 = 448
  s.red = reinterpret_cast<float *>(misc + 704);            // 64 * 4 = 256
  s.flags = reinterpret_cast<int *>(misc + 960);            // 16 ints
  s.acc_bar = s.empty + 8;                                  // entries 8.. of the empty-barrier array are unused (<= 8 stages)
  s.tmem_holder = reinterpret_cast<uint32_t *>(s.empty + 9);
  return s;
}

struct LinearState {   // position of the compute warps in the weight stage ring
  int stage;
  uint32_t phase;
  uint32_t acc_phase;   // parity of the next completion of the tcgen05 accumulator barrier
};

struct Ctx {
  const KernelParams &P;
  Smem s;
  unsigned long long iteration;
  uint64_t deadline_ns;   // absolute globaltimer value after which waits give up
  int worker;
  uint32_t tmem_base;     // tensor-memory address of column 0 (general instantiation, graphs with tcgen05 tasks)
};

// ---------------------------------------------------------------------------
// bounded waits
// ---------------------------------------------------------------------------
__device__ __noinline__ void report_timeout(DeviceStatus *st, int worker, int where, int task) {
  if (atomicCAS(&st->error, 0, -4) == 0) {
    st->where = where;
    st->worker = worker;
    st->task = task;
    __threadfence();
  }
}

// Returns false when the wait was abandoned (timeout here or abort raised elsewhere).
__device__ __forceinline__ bool wait_mbar(const Ctx &c, uint64_t *bar, uint32_t parity, int task) {
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 0x3ff) == 0) {
      if (ld_volatile_i32(&c.P.status->error) != 0) return false;
      if (globaltimer_ns() > c.deadline_ns) {
        report_timeout(c.P.status, c.worker, 2, task);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ bool wait_counter(const Ctx &c, const unsigned long long *ctr,
                                             unsigned long long need, bool sys_scope, int where, int task) {
  uint32_t polls = 0;
  while (true) {
    unsigned long long v = sys_scope ? ld_acquire_sys(ctr) : ld_acquire_gpu(ctr);
    if (v >= need) return true;
    if ((++polls & 0xff) == 0) {
      if (ld_volatile_i32(&c.P.status->error) != 0) return false;
      if (globaltimer_ns() > c.deadline_ns) {
        report_timeout(c.P.status, c.worker, where, task);
        return false;
      }
    }
    if (c.P.poll_sleep_ns) __nanosleep(c.P.poll_sleep_ns);
  }
}

template <bool GENERAL>
__device__ void prefetch_attention_kv_l2(const Ctx &c, const TaskDesc *d, int lane, int task);

// ---------------------------------------------------------------------------
// weight streamer (warp 8)
// ---------------------------------------------------------------------------
// A linear task streams its weight panel [n0, n1) x K as chunks of 16 rows x KC columns (KC <= 1024):
// one cp.async.bulk per row segment, rows padded by 16 bytes in shared memory so that ldmatrix reads
// are bank-conflict free.  Order: k tile (activation tile) -> 16-row group -> k chunk.
template <bool GENERAL>
__device__ void streamer_loop(const Ctx &c, int t_begin, int t_end) {
  const KernelParams &P = c.P;
  const int lane = threadIdx.x & 31;
  const uint64_t policy = l2_policy_evict_first();
  const int NST = P.num_stages;
  uint32_t issued = 0;
  int s = 0;
  uint32_t ph = 0;
  int s_land = 0;          // oldest chunk that may still be in flight (pacing)
  uint32_t ph_land = 0;
  const uint32_t max_inflight = (uint32_t)P.max_inflight;
  bool ok = true;
  // The whole warp walks the task list; lane 0 owns the barrier traffic, lane r copies row r of a chunk.
  for (int t = t_begin; t < t_end && ok; ++t) {
    const TaskDesc *d = &P.tasks[t];
    if (d->type == TASK_ATTENTION && P.kv_l2_prefetch) prefetch_attention_kv_l2<GENERAL>(c, d, lane, t);
    if (d->type != TASK_LINEAR && !(GENERAL && d->type == TASK_MOE_GEMM)) continue;
    if (d->flags & TF_STREAM_AFTER_DEP) {
      if (lane == 0)
        for (int i = 0; i < kMaxDeps && ok; ++i)
          if (d->dep_event[i] >= 0)
            ok = wait_counter(c, &P.counters[d->dep_event[i]], (unsigned long long)d->dep_need[i] * c.iteration,
                              false, 1, t);
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      if (!ok) break;
      fence_proxy_async_all();   // the weights were written through the generic proxy; the bulk copies read through the async proxy
    }
    if (GENERAL && (d->flags & TF_TC)) {
      // tcgen05 path: one tensor-map TMA per ring slot brings a box of {64 columns, RB rows, nkb k blocks} of the
      // task's own row panel (rows past the panel are filled with zeros and cost no HBM traffic) in the
      // 128-byte-swizzled layout the MMA reads.  Order: k tile -> row tile -> k blocks.
      const uint8_t *tmap = reinterpret_cast<const uint8_t *>(P.tmaps) + (size_t)d->a[L_TMAP] * 128;
      const int rows = d->a[L_N1] - d->a[L_N0], RB = d->a[L_ROWS];
      const int kbe = (d->flags & TF_FP8) ? 2 * kTcKBlock : kTcKBlock;   // elements of one 128-byte k block
      const int nkb = d->a[L_KC] / kbe, kbt = d->a[L_KT] / kbe, kball = d->a[L_K] / kbe;
      const int tiles = (rows + RB - 1) / RB;
      const uint32_t tx = (uint32_t)(nkb * RB * 128);
      for (int kb_t = 0; kb_t < kball && ok; kb_t += kbt)
        for (int tile = 0; tile < tiles && ok; ++tile)
          for (int kb = 0; kb < kbt; kb += nkb) {
            if (lane == 0) {
              ok = wait_mbar(c, &c.s.empty[s], ph ^ 1u, t);
              if (ok) {
                mbar_arrive_expect_tx(&c.s.full[s], tx);
                tma_load_3d(c.s.stages + (size_t)s * P.stage_bytes, tmap, 0, tile * RB, kb_t + kb, &c.s.full[s], policy);
              }
            }
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            if (!ok) break;
            ++issued;
            if (++s == NST) { s = 0; ph ^= 1u; }
          }
      continue;
    }
    const uint8_t *W = reinterpret_cast<const uint8_t *>(d->p[0]);
    const int n0 = d->a[L_N0], n1 = d->a[L_N1], K = d->a[L_K], ldw = d->a[L_LDW];
    const int KT = d->a[L_KT], KC = d->a[L_KC], R = d->a[L_ROWS];
    const uint32_t esz = (GENERAL && (d->flags & TF_FP8)) ? 1u : 2u;   // e4m3 or bf16 weights
    const uint32_t seg_bytes = (uint32_t)KC * esz;
    const uint32_t row_stride = seg_bytes + kRowPadBytes;
    // an expert task repeats the panel loop once per active expert (the list is final: the task waited for it)
    int reps = 1;
    const int *act = nullptr;
    if (GENERAL && d->type == TASK_MOE_GEMM) {
      act = reinterpret_cast<const int *>(d->p[5]);
      reps = min(__ldcg(&act[d->a[M_NEXP]]), d->a[M_NEXP]);
    }
    for (int rep = 0; rep < reps && ok; ++rep) {
    const uint8_t *Wp = W;
    if (GENERAL && act != nullptr) Wp = W + (size_t)__ldcg(&act[rep]) * (size_t)d->a[M_ESTRIDE] * esz;
    for (int kt = 0; kt < K && ok; kt += KT) {
      for (int r0 = n0; r0 < n1 && ok; r0 += R) {
        const int rows = min(R, n1 - r0);
        const uint8_t *src_row = Wp + ((size_t)(r0 + lane) * ldw + kt) * esz;   // valid for lane < rows
        for (int kc = 0; kc < KT; kc += KC) {
          if (lane == 0) {
            ok = wait_mbar(c, &c.s.empty[s], ph ^ 1u, t);
            // pacing: keep at most max_inflight chunks between "issued" and "landed", so that the
            // latency-critical loads and stores of the compute warps do not queue behind a full ring
            if (ok && max_inflight < (uint32_t)NST && issued >= max_inflight) {
              ok = wait_mbar(c, &c.s.full[s_land], ph_land, t);
              if (++s_land == NST) { s_land = 0; ph_land ^= 1u; }
            }
            // quiet mode: while the compute warps run a latency-bound task (attention), hold the weight
            // stream back so that their loads do not wait behind megabytes of queued weight traffic
            if (ok && P.quiet_streaming) {
              uint32_t polls = 0;
              while (*reinterpret_cast<volatile int *>(&c.s.flags[2]) != 0) {
                __nanosleep(100);
                if ((++polls & 0xff) == 0 && (ld_volatile_i32(&P.status->error) != 0 || globaltimer_ns() > c.deadline_ns)) break;
              }
            }
            if (ok) mbar_arrive_expect_tx(&c.s.full[s], (uint32_t)rows * seg_bytes);
          }
          ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
          if (!ok) break;
          if (lane < rows)
            bulk_g2s(c.s.stages + (size_t)s * P.stage_bytes + (size_t)lane * row_stride, src_row + (size_t)kc * esz,
                     seg_bytes, &c.s.full[s], policy);
          ++issued;
          if (++s == NST) { s = 0; ph ^= 1u; }
        }
      }
    }
    }
  }
  // Drain: every copy this warp issued must have landed before the CTA may exit.
  if (lane == 0) {
    const uint32_t pending = issued < (uint32_t)NST ? issued : (uint32_t)NST;
    for (uint32_t q = 0; q < pending; ++q) {
      if (--s < 0) { s = NST - 1; ph ^= 1u; }
      uint32_t polls = 0;
      while (!mbar_try_wait(&c.s.full[s], ph)) {
        if (++polls > (1u << 24)) break;   // copies in flight always complete; the bound only guards the loop
      }
    }
  }
  __syncwarp();
}

// ---------------------------------------------------------------------------
// TASK_LINEAR: weight-streaming skinny GEMM for up to 8 tokens on mma.sync m16n8k16
// (16 weight rows x 16 k per instruction, the tokens are the n dimension)
// ---------------------------------------------------------------------------
__device__ __forceinline__ int active_tokens(const KernelParams &P) {
  if (P.test_mode || P.meta.qo_indptr == nullptr) return P.max_num_batched_tokens;
  return __ldcg(&P.meta.qo_indptr[P.max_num_batched_requests]);
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 16-bit sequence number of an allreduce instance: never 0 (a zeroed inbox is invalid).  Two instances carry the same
// number AND use the same inbox buffer when they are a multiple of 131070 (= lcm(65535, 2)) instances apart.  Rows
// [0, active tokens) of a buffer are rewritten by every instance that uses it, so only a token row that sat idle
// since exactly such an instance and becomes active again could show a consumer a stale word that passes the check.
// The batching task therefore clears the rows that go idle when the number of active tokens drops (run_batch; race
// free: every word of the finished iteration has been consumed, and peers push only rows below the new count), which
// leaves no stale sequence number behind.  Graphs without a batching task keep a fixed token count (test mode) or take
// it from the caller (online_notoken: a caller that shrinks and regrows the batch within 131070 / allreduces-per-
// iteration iterations of the same run is not covered).
__device__ __forceinline__ uint32_t ll_seq(unsigned long long iteration, int n_ar, int ar_idx) {
  return (uint32_t)((iteration * (unsigned long long)n_ar + (unsigned long long)ar_idx) % 65535ull) + 1u;
}

// fast silu: x * sigmoid(x) with ex2.approx based exp and approximate divide (error far below bf16 rounding)
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Stage the activation tile [B, KT] (bf16, rows padded by 16 bytes) for k range [k0, k0 + KT).
// `gpre` holds this thread's first two gamma vectors, loaded before the dependency wait.
// Address of 16-byte vector v (k elements 8v .. 8v + 7 of the tile) of token row b.  MODE 0 / 1: row-major rows
// padded by 16 bytes (mma.sync fragments); MODE 2: the tcgen05 operand layout -- blocks of 64 columns, each block
// [token rows][128 bytes] with the 16-byte chunks of a row XOR-swizzled by (row & 7) (128-byte swizzle, K-major).
template <int MODE>
__device__ __forceinline__ uint8_t *x_vec(uint8_t *xs, int b, int v, int xstride, int np) {
  if (MODE == 2)
    return xs + (size_t)(v >> 3) * (size_t)(np * 128) + (size_t)b * 128 + (size_t)(((v & 7) ^ (b & 7)) << 4);
  return xs + (size_t)b * xstride + (size_t)v * 16;
}

// Fused tensor-parallel allreduce, consumer side, with every rank's words of a vector requested before any of them
// is examined: a vector costs one L2 round trip (plus re-polls of the ranks that had not arrived) instead of one per
// rank.  Returns the thread's sum of squares over the vectors it wrote; `good` turns false when a wait ran out.
template <int MODE>
__device__ __forceinline__ float gather_row(const Ctx &c, const TaskDesc &d, const uint32_t *inbox, uint32_t seq, int b, int k0,
                                            int vec_per_row, int xstride, int np, bool &good) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x;
  const int K = d.a[L_K], slot = d.a[L_G_SLOT], W = P.world_size;
  const __nv_bfloat16 *res = reinterpret_cast<const __nv_bfloat16 *>(d.p[6]);
  __nv_bfloat16 *yout = reinterpret_cast<__nv_bfloat16 *>(d.p[7]);
  float ss = 0.f;
  for (int v = tid; v < vec_per_row && good; v += kConsumerThreads) {
    const uint32_t *wp = inbox + (size_t)b * K + k0 + v * 8;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    // four ranks per trip: their eight 16-byte loads are in flight together; the quad is re-read until all of it has
    // arrived and only then added, in rank order (every rank forms the same sum)
#pragma unroll
    for (int h = 0; h < kMaxWorld; h += 4) {
      if (h >= W) break;
      uint4 w0[4], w1[4];
      uint32_t polls = 0;
      while (true) {
        bool all = true;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (h + i < W) {
            const uint32_t *q = wp + (size_t)(h + i) * slot;
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(w0[i].x), "=r"(w0[i].y), "=r"(w0[i].z), "=r"(w0[i].w) : "l"(q) : "memory");
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(w1[i].x), "=r"(w1[i].y), "=r"(w1[i].z), "=r"(w1[i].w) : "l"(q + 4) : "memory");
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (h + i < W)
            all = all && (w0[i].x >> 16) == seq && (w0[i].y >> 16) == seq && (w0[i].z >> 16) == seq && (w0[i].w >> 16) == seq &&
                  (w1[i].x >> 16) == seq && (w1[i].y >> 16) == seq && (w1[i].z >> 16) == seq && (w1[i].w >> 16) == seq;
        }
        if (all) break;
        if ((++polls & 0x3f) == 0) {
          if (ld_volatile_i32(&P.status->error) != 0) { good = false; break; }
          if (globaltimer_ns() > c.deadline_ns) {
            report_timeout(P.status, c.worker, 3, h);
            good = false;
            break;
          }
        }
      }
      if (!good) break;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (h + i < W) {
          const uint32_t ww[8] = {w0[i].x, w0[i].y, w0[i].z, w0[i].w, w1[i].x, w1[i].y, w1[i].z, w1[i].w};
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += __uint_as_float(ww[e] << 16);
        }
      }
    }
    if (!good) break;
    if (res) {
      const uint4 rv = __ldcg(reinterpret_cast<const uint4 *>(res + (size_t)b * d.a[L_G_LDRES] + k0) + v);
      const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += bf16_lo(rw[q]);
        acc[2 * q + 1] += bf16_hi(rw[q]);
      }
    }
    uint32_t ow[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      ow[q] = pack_bf16(acc[2 * q], acc[2 * q + 1]);
      const float a = bf16_lo(ow[q]), e = bf16_hi(ow[q]);
      ss += a * a + e * e;
    }
    const uint4 o4 = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    *reinterpret_cast<uint4 *>(x_vec<MODE>(c.s.xtile, b, v, xstride, np)) = o4;
    reinterpret_cast<uint4 *>(yout + (size_t)b * d.a[L_G_LDOUT] + k0)[v] = o4;
  }
  return ss;
}

template <int MODE, bool TPX = false>
__device__ void stage_x(const Ctx &c, const TaskDesc &d, int B, int k0, int KT, const uint4 (&gpre)[2]) {
  constexpr bool WIDE = MODE != 0;
  const int np = c.P.tc_tokens;
  const int tid = threadIdx.x;
  const int K = d.a[L_K];
  const int ldx = d.a[L_LDX];
  const int pro = d.a[L_PRO];
  const int vec_per_row = KT / 8;
  const int xstride = KT * 2 + kRowPadBytes;   // bytes
  uint8_t *xs = c.s.xtile;
  // per-token, per-warp sums of squares: 8 x 8 floats, or up to 64 x 8 in the partial-sum area (idle while the
  // activation tile is staged)
  float *red = WIDE ? c.s.partial : c.s.red;
  const __nv_bfloat16 *src = reinterpret_cast<const __nv_bfloat16 *>(d.p[1]);
  if (d.a[L_GATHER] > 0) {
    // Fused tensor-parallel allreduce: every rank pushed {bf16 partial, sequence} words for this allreduce
    // instance into our inbox.  Poll until all words of a vector carry the expected sequence number, sum the
    // ranks in rank order in fp32, add the residual, round once: that is the reduced activation row.  It is
    // staged in shared memory for this task and written to its tensor (every task writes the same values).
    const KernelParams &P = c.P;
    const int ar = d.a[L_GATHER] - 1;
    const unsigned long long inst = c.iteration * (unsigned)d.a[L_NAR] + (unsigned)ar;
    const uint32_t seq = ll_seq(c.iteration, d.a[L_NAR], ar);
    const uint32_t *inbox = reinterpret_cast<const uint32_t *>(P.peer_inbox[P.rank]) + (size_t)d.p[5] +
                            (size_t)(inst & 1ull) * (size_t)d.a[L_PARSTRIDE];
    const __nv_bfloat16 *res = reinterpret_cast<const __nv_bfloat16 *>(d.p[6]);
    __nv_bfloat16 *yout = reinterpret_cast<__nv_bfloat16 *>(d.p[7]);
    const int slot = d.a[L_G_SLOT];
    const int warp = tid >> 5, lane = tid & 31;
    bool good = true;
    for (int b = 0; b < B; ++b) {
      float ss = 0.f;
      if (TPX && MODE == 0) ss = gather_row<MODE>(c, d, inbox, seq, b, k0, vec_per_row, xstride, np, good);
      for (int v = tid; !(TPX && MODE == 0) && v < vec_per_row; v += kConsumerThreads) {
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int r = 0; r < P.world_size; ++r) {
          const uint32_t *wp = inbox + (size_t)r * slot + (size_t)b * K + k0 + v * 8;
          uint4 w0, w1;
          uint32_t polls = 0;
          while (true) {
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(w0.x), "=r"(w0.y), "=r"(w0.z), "=r"(w0.w) : "l"(wp) : "memory");
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(w1.x), "=r"(w1.y), "=r"(w1.z), "=r"(w1.w) : "l"(wp + 4) : "memory");
            const bool ok8 = (w0.x >> 16) == seq && (w0.y >> 16) == seq && (w0.z >> 16) == seq && (w0.w >> 16) == seq &&
                             (w1.x >> 16) == seq && (w1.y >> 16) == seq && (w1.z >> 16) == seq && (w1.w >> 16) == seq;
            if (ok8) break;
            if ((++polls & 0xff) == 0) {
              if (ld_volatile_i32(&P.status->error) != 0) { good = false; break; }
              if (globaltimer_ns() > c.deadline_ns) {
                report_timeout(P.status, c.worker, 3, r);
                good = false;
                break;
              }
            }
          }
          if (!good) break;
          const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += __uint_as_float(ww[e] << 16);
        }
        uint32_t ow[4];
        if (res) {
          const uint4 rv = __ldcg(reinterpret_cast<const uint4 *>(res + (size_t)b * d.a[L_G_LDRES] + k0) + v);
          const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            acc[2 * q] += bf16_lo(rw[q]);
            acc[2 * q + 1] += bf16_hi(rw[q]);
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          ow[q] = pack_bf16(acc[2 * q], acc[2 * q + 1]);
          const float a = bf16_lo(ow[q]), e = bf16_hi(ow[q]);
          ss += a * a + e * e;
        }
        const uint4 o4 = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        *reinterpret_cast<uint4 *>(x_vec<MODE>(xs, b, v, xstride, np)) = o4;
        reinterpret_cast<uint4 *>(yout + (size_t)b * d.a[L_G_LDOUT] + k0)[v] = o4;
      }
      if (!WIDE || pro == PRO_RMSNORM) {   // (whole row staged: the partial-sum area is not holding sums of a previous k tile)
        ss = warp_sum(ss);
        if (lane == 0) red[b * 8 + warp] = ss;
      }
    }
    if (!good) c.s.flags[0] = 1;
    consumer_sync();
    if (pro != PRO_RMSNORM) return;
    const float eps = __int_as_float(d.a[L_EPS]);
    const __nv_bfloat16 *gam = reinterpret_cast<const __nv_bfloat16 *>(d.p[4]);
    for (int b = 0; b < B; ++b) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) tot += red[b * 8 + w];
      const float inv = rsqrtf(tot / (float)K + eps);
      int it = 0;
      for (int v = tid; v < vec_per_row; v += kConsumerThreads, ++it) {
        uint4 *xp = reinterpret_cast<uint4 *>(x_vec<MODE>(xs, b, v, xstride, np));
        const uint4 xv = *xp;
        const uint4 gv = (it < 2) ? gpre[it] : __ldg(reinterpret_cast<const uint4 *>(gam + k0) + v);
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
        uint32_t ow[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
          ow[q] = pack_bf16(bf16_lo(xw[q]) * inv * bf16_lo(gw[q]), bf16_hi(xw[q]) * inv * bf16_hi(gw[q]));
        *xp = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
    }
    consumer_sync();
    return;
  }
  if (pro == PRO_SILU_MUL) {
    const int groups = d.a[L_GROUPS];
    const int per = K / groups;   // activation columns per interleave group
    for (int b = 0; b < B; ++b) {
      for (int v = tid; v < vec_per_row; v += kConsumerThreads) {
        const int j = k0 + v * 8;
        const int g = j / per, off = j - g * per;
        const __nv_bfloat16 *gp = src + (size_t)b * ldx + (size_t)g * 2 * per + off;
        const uint4 gv = __ldcg(reinterpret_cast<const uint4 *>(gp));
        const uint4 uv = __ldcg(reinterpret_cast<const uint4 *>(gp + per));
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
        const uint32_t uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t ow[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float a0 = round_bf16(silu_f(bf16_lo(gw[q])));
          const float a1 = round_bf16(silu_f(bf16_hi(gw[q])));
          ow[q] = pack_bf16(a0 * bf16_lo(uw[q]), a1 * bf16_hi(uw[q]));
        }
        *reinterpret_cast<uint4 *>(x_vec<MODE>(xs, b, v, xstride, np)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
    }
    consumer_sync();
    return;
  }
  if (WIDE && (pro == PRO_PLAIN || pro == PRO_RMSNORM)) {
    // many tokens: asynchronous 16-byte copies straight into shared memory (all in flight, no registers held)
    for (int b = 0; b < B; ++b)
      for (int v = tid; v < vec_per_row; v += kConsumerThreads)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(x_vec<MODE>(xs, b, v, xstride, np))),
                     "l"(reinterpret_cast<const uint4 *>(src + (size_t)b * ldx + k0) + v)
                     : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    consumer_sync();
    if (pro == PRO_PLAIN) return;
    // RMSNorm in place.  Pass 1: one warp per token sums the squares and leaves 1 / rms in shared memory.  Pass 2:
    // a thread owns vector positions v = tid, tid + 256, ... of EVERY token, so that gamma (fetched before the
    // dependency wait for the first two positions) sits in registers and no global load is left in the loop.
    const int warp = tid >> 5, lane = tid & 31;
    const float eps = __int_as_float(d.a[L_EPS]);
    const __nv_bfloat16 *gam = reinterpret_cast<const __nv_bfloat16 *>(d.p[4]);
    for (int b = warp; b < B; b += 8) {
      float ss = 0.f;
      for (int v = lane; v < vec_per_row; v += 32) {
        const uint4 xv = *reinterpret_cast<const uint4 *>(x_vec<MODE>(xs, b, v, xstride, np));
        const uint32_t w[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float a = bf16_lo(w[q]), e = bf16_hi(w[q]);
          ss += a * a + e * e;
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) red[b] = rsqrtf(ss / (float)K + eps);
    }
    consumer_sync();
    int it = 0;
    for (int v = tid; v < vec_per_row; v += kConsumerThreads, ++it) {
      const uint4 gv = (it < 2) ? gpre[it] : __ldg(reinterpret_cast<const uint4 *>(gam + k0) + v);
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
      float gf[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) { gf[2 * q] = bf16_lo(gw[q]); gf[2 * q + 1] = bf16_hi(gw[q]); }
#pragma unroll 4
      for (int b = 0; b < B; ++b) {
        const float inv = red[b];
        uint4 *xp = reinterpret_cast<uint4 *>(x_vec<MODE>(xs, b, v, xstride, np));
        const uint4 xv = *xp;
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
        uint32_t ow[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
          ow[q] = pack_bf16(bf16_lo(xw[q]) * inv * gf[2 * q], bf16_hi(xw[q]) * inv * gf[2 * q + 1]);
        *xp = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
    }
    consumer_sync();
    return;
  }
  if (pro != PRO_RMSNORM) {
    for (int b = 0; b < B; ++b)
      for (int v = tid; v < vec_per_row; v += kConsumerThreads)
        *reinterpret_cast<uint4 *>(x_vec<MODE>(xs, b, v, xstride, np)) =
            __ldcg(reinterpret_cast<const uint4 *>(src + (size_t)b * ldx + k0) + v);
    consumer_sync();
    return;
  }
  // RMSNorm over the full row (the builder guarantees KT == K for this prologue).
  const int warp = tid >> 5, lane = tid & 31;
  for (int b = 0; b < B; ++b) {
    float ss = 0.f;
    for (int v = tid; v < vec_per_row; v += kConsumerThreads) {
      const uint4 xv = __ldcg(reinterpret_cast<const uint4 *>(src + (size_t)b * ldx + k0) + v);
      *reinterpret_cast<uint4 *>(x_vec<MODE>(xs, b, v, xstride, np)) = xv;
      const uint32_t w[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float a = bf16_lo(w[q]), e = bf16_hi(w[q]);
        ss += a * a + e * e;
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[b * 8 + warp] = ss;
  }
  consumer_sync();
  const float eps = __int_as_float(d.a[L_EPS]);
  const __nv_bfloat16 *gam = reinterpret_cast<const __nv_bfloat16 *>(d.p[4]);
  for (int b = 0; b < B; ++b) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[b * 8 + w];
    const float inv = rsqrtf(tot / (float)K + eps);
    int it = 0;
    for (int v = tid; v < vec_per_row; v += kConsumerThreads, ++it) {
      uint4 *xp = reinterpret_cast<uint4 *>(x_vec<MODE>(xs, b, v, xstride, np));
      const uint4 xv = *xp;
      const uint4 gv = (it < 2) ? gpre[it] : __ldg(reinterpret_cast<const uint4 *>(gam + k0) + v);
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
      uint32_t ow[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        ow[q] = pack_bf16(bf16_lo(xw[q]) * inv * bf16_lo(gw[q]), bf16_hi(xw[q]) * inv * bf16_hi(gw[q]));
      *xp = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
  }
  consumer_sync();
}

// Sum the 8 warps' partial tiles of one 16-row group and run the epilogue for its rows.
// WIDE = false: at most 8 tokens, every warp holds the same token tile (the batch-1 hot path, all constants);
// WIDE = true: warp w holds token tile w % NT (8 tokens each) and every (8 / NT)-th k step.
template <bool WIDE>
__device__ __forceinline__ void linear_output(const Ctx &c, const TaskDesc &d, int NT, int r0, int rows,
                                              const float *part, int item);

template <bool WIDE>
__device__ __forceinline__ void linear_group_epilogue(const Ctx &c, const TaskDesc &d, int B, int NT, int r0, int rows,
                                                      const float *part) {
  if (!WIDE) {
    const int tid = threadIdx.x;
    if (tid < 128 && (tid >> 4) < B) linear_output<false>(c, d, 1, r0, rows, part, tid);
  } else {
    for (int item = threadIdx.x; item < B * 16; item += kConsumerThreads) linear_output<true>(c, d, NT, r0, rows, part, item);
  }
}

template <bool WIDE>
__device__ __forceinline__ void linear_output(const Ctx &c, const TaskDesc &d, int NT, int r0, int rows,
                                              const float *part, int item) {
  const KernelParams &P = c.P;
  const int b = item >> 4, r = item & 15;
  if (r >= rows) return;
  float v = 0.f;
  if (WIDE) {
    for (int w = b >> 3; w < 8; w += NT) v += part[(w * 16 + r) * 8 + (b & 7)];
  } else {
#pragma unroll
    for (int w = 0; w < 8; ++w) v += part[(w * 16 + r) * 8 + b];
  }
  const int epi = d.a[L_EPI];
  const int col = r0 + r;
  if (epi == EPI_PUSH_LL) {
    // one 32-bit word per element: bf16 partial sum in the low half, sequence number in the high half
    const int N = d.a[L_N];
    const unsigned long long inst = c.iteration * (unsigned)d.a[L_NAR] + (unsigned)d.a[L_ARIDX];
    const size_t off = (size_t)d.p[5] + (size_t)(inst & 1ull) * (size_t)d.a[L_PARSTRIDE] +
                       (size_t)P.rank * (size_t)d.a[L_SLOT] + (size_t)b * N + col;
    const __nv_bfloat16 hv = __float2bfloat16_rn(v);
    const uint32_t word = (uint32_t)(*reinterpret_cast<const unsigned short *>(&hv)) |
                          (ll_seq(c.iteration, d.a[L_NAR], d.a[L_ARIDX]) << 16);
    for (int peer = 0; peer < P.world_size; ++peer)
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<uint32_t *>(P.peer_inbox[peer]) + off),
                   "r"(word)
                   : "memory");
  } else if (epi == EPI_PUSH_F32) {
    const int N = d.a[L_N];
    const size_t parity = (size_t)((c.iteration * (unsigned)d.a[L_NAR] + (unsigned)d.a[L_ARIDX]) & 1ull);
    const size_t off = (size_t)d.p[5] + parity * (size_t)d.a[L_PARSTRIDE] + (size_t)P.rank * (size_t)d.a[L_SLOT] +
                       (size_t)b * N + col;
    for (int peer = 0; peer < P.world_size; ++peer) P.peer_inbox[peer][off] = v;
  } else if (epi == EPI_SILU_PAIR) {
    // rows come as [gate, gate, up, up]: the threads on gate rows finish the pair
    if ((r & 2) == 0) {
      float u = 0.f;
      if (WIDE) {
        for (int w = b >> 3; w < 8; w += NT) u += part[(w * 16 + r + 2) * 8 + (b & 7)];
      } else {
#pragma unroll
        for (int w = 0; w < 8; ++w) u += part[(w * 16 + r + 2) * 8 + b];
      }
      const float gv = round_bf16(v);
      const float a = round_bf16(silu_f(gv));
      __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
      out[(size_t)b * d.a[L_LDO] + ((col >> 2) << 1) + (r & 1)] = __float2bfloat16_rn(a * round_bf16(u));
    }
  } else {
    __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
    if (epi == EPI_RESIDUAL) {
      const __nv_bfloat16 *res = reinterpret_cast<const __nv_bfloat16 *>(d.p[3]);
      v += bf16_to_f(__ldcg(&res[(size_t)b * d.a[L_LDR] + col]));
    }
    out[(size_t)b * d.a[L_LDO] + col] = __float2bfloat16_rn(v);
  }
}

template <bool WIDE, bool TPX = false>
__device__ __forceinline__ void run_linear(const Ctx &c, const TaskDesc &d, LinearState &ls, int task,
                                           const uint4 (&gpre)[2], bool ok) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int B = ok ? min(active_tokens(P), WIDE ? kMaxLinearTokens : 8) : 0;
  const int NT = !WIDE || B <= 8 ? 1 : (B <= 16 ? 2 : (B <= 32 ? 4 : 8));   // token tiles of 8
  const int nt = WIDE ? warp % NT : 0, ks = WIDE ? warp / NT : warp, kstride = WIDE ? 8 / NT : 8;
  const int n0 = d.a[L_N0], n1 = d.a[L_N1], K = d.a[L_K];
  const int KT = d.a[L_KT], KC = d.a[L_KC], R = d.a[L_ROWS];
  const int NST = P.num_stages;
  const int steps = KC / 16;
  const uint32_t row_stride = (uint32_t)KC * 2u + kRowPadBytes;
  const uint32_t xstride = (uint32_t)KT * 2u + kRowPadBytes;
  const int g = lane >> 2, q = lane & 3;
  const bool tok_valid = nt * 8 + g < B;
  const bool multi_tile = KT < K;          // accumulate across k tiles in shared memory (task has <= 2 groups)
  // lanes 0-15 address the 16 rows of the m-tile; with 8-row chunks rows 8-15 alias rows 0-7 (their results are unused)
  const uint32_t a_lane_off = (uint32_t)(lane & (R - 1)) * row_stride + (uint32_t)(lane >> 4) * 16u;
  const uint32_t x_lane_base =
      smem_u32(c.s.xtile) + (uint32_t)(tok_valid ? nt * 8 + g : 0) * xstride + (uint32_t)q * 4u;
  const bool prof = P.profiler != nullptr && (uint64_t)(task + 1) * 8 <= P.profiler_entries;
  int group_seq = 0;
  int nchunk = 0;
  for (int kt = 0; kt < K; kt += KT) {
    if (B > 0 && !((d.flags & TF_SAME_X_AS_PREV) && !multi_tile)) {
      if (kt > 0) consumer_sync();   // everyone is done reading the previous tile
      stage_x<WIDE ? 1 : 0, TPX>(c, d, B, kt, KT, gpre);
    }
    if (tid == 0 && prof && kt == 0) P.profiler[(size_t)task * 8 + 4] = globaltimer_ns();
    int gi = 0;
    for (int r0 = n0; r0 < n1; r0 += R, ++gi) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      float acc2[4] = {0.f, 0.f, 0.f, 0.f};   // second accumulator chain: back-to-back mma do not serialise
      for (int kc = 0; kc < KT; kc += KC) {
        const int s = ls.stage;
        const uint32_t ph = ls.phase;
        if (++ls.stage == NST) { ls.stage = 0; ls.phase ^= 1u; }
        if (ok) ok = wait_mbar(c, &c.s.full[s], ph, task);
        if (ok && B > 0) {
          const uint32_t a_base = smem_u32(c.s.stages + (size_t)s * P.stage_bytes) + a_lane_off;
          const uint32_t x_base = x_lane_base + (uint32_t)kc * 2u;
          // this warp's k steps are warp, warp + 8, ...; fetch the fragments of four steps, then issue their mma
          const int nj = WIDE ? (steps - ks + kstride - 1) / kstride : (steps - warp + 7) >> 3;
          for (int j0 = 0; j0 < nj; j0 += 4) {
            uint32_t a[4][4], b[4][2];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (j0 + u < nj) {
                const uint32_t o = (uint32_t)(ks + kstride * (j0 + u)) * 32u;
                ldmatrix_x4(a[u], a_base + o);
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(b[u][0]) : "r"(x_base + o));
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(b[u][1]) : "r"(x_base + o + 16u));
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (j0 + u < nj) {
                if (!tok_valid) b[u][0] = b[u][1] = 0u;   // token columns beyond the batch contribute nothing
                if (u & 1) mma_bf16_16816(acc2, a[u], b[u][0], b[u][1]);
                else mma_bf16_16816(acc, a[u], b[u][0], b[u][1]);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&c.s.empty[s]);
        if (tid == 0 && prof) {
          ++nchunk;
          if (nchunk == 1) P.profiler[(size_t)task * 8 + 6] = globaltimer_ns();
          if (nchunk == 6) P.profiler[(size_t)task * 8 + 7] = globaltimer_ns();
        }
      }
      if (B > 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] += acc2[i];
        // this warp's 16 x 8 partial tile -> shared memory
        float *part = c.s.partial + (size_t)((multi_tile ? gi : group_seq) & 1) * (8 * 16 * 8);
        float *mine = part + (size_t)warp * (16 * 8);
        float2 *p0 = reinterpret_cast<float2 *>(mine + g * 8 + q * 2);
        float2 *p1 = reinterpret_cast<float2 *>(mine + (g + 8) * 8 + q * 2);
        if (multi_tile && kt > 0) {
          float2 o0 = *p0, o1 = *p1;
          *p0 = make_float2(o0.x + acc[0], o0.y + acc[1]);
          *p1 = make_float2(o1.x + acc[2], o1.y + acc[3]);
        } else {
          *p0 = make_float2(acc[0], acc[1]);
          *p1 = make_float2(acc[2], acc[3]);
        }
        if (!multi_tile) {
          consumer_sync();
          linear_group_epilogue<WIDE>(c, d, B, NT, r0, min(R, n1 - r0), part);
        }
      }
      ++group_seq;
    }
  }
  if (!ok) c.s.flags[0] = 1;
  if (tid == 0 && prof) P.profiler[(size_t)task * 8 + 5] = globaltimer_ns();
  if (B > 0 && multi_tile) {
    consumer_sync();
    int gi = 0;
    for (int r0 = n0; r0 < n1; r0 += R, ++gi)
      linear_group_epilogue<WIDE>(c, d, B, NT, r0, min(R, n1 - r0), c.s.partial + (size_t)(gi & 1) * (8 * 16 * 8));
  }
}

// ---------------------------------------------------------------------------
// TASK_LINEAR on the tensor path (general instantiation, graphs with more than 8 batched tokens): the weights are
// the M operand (swap-AB, as in include/mirage/persistent_kernel/tasks/blackwell/linear_sm100_mpk.cuh:31-735),
// 128 rows per tcgen05.mma, the batched tokens the N operand (16 .. 64), fp32 accumulators in tensor memory.
// The task's rows are cut into tiles of RB <= 128 rows; tile t accumulates into columns [t * NP, t * NP + N) over
// ALL k tiles of the activation, so the weights stream exactly once and the activation tile is staged once per k
// tile.  Thread 0 issues the MMAs as ring slots fill and hands each slot back with tcgen05.commit; after the last
// k block all eight warps read their lane quadrant of the accumulators (tcgen05.ld) and run the epilogue.
// ---------------------------------------------------------------------------
// Everything the epilogue of a tcgen05 linear task needs from its descriptor, read once into registers: the
// descriptor lives in shared memory behind a generic reference, and a load from it may not move across the global
// stores of the epilogue (they could alias), so reading it per element costs a chain of dependent loads every time.
struct EmitArgs {
  int epi, ldo, world;
  __nv_bfloat16 *out;
  size_t push_off;      // element offset of (token 0, column 0) of this rank's slot in an inbox buffer
  int push_n;           // row length of the pushed matrix
  uint32_t seq_hi;      // sequence number of the allreduce instance, already shifted to the high half
};

__device__ __forceinline__ EmitArgs emit_args(const Ctx &c, const TaskDesc &d) {
  EmitArgs e;
  e.epi = d.a[L_EPI];
  e.ldo = d.a[L_LDO];
  e.world = c.P.world_size;
  e.out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  const unsigned long long inst = c.iteration * (unsigned)d.a[L_NAR] + (unsigned)d.a[L_ARIDX];
  e.push_off = (size_t)d.p[5] + (size_t)(inst & 1ull) * (size_t)d.a[L_PARSTRIDE] + (size_t)c.P.rank * (size_t)d.a[L_SLOT];
  e.push_n = d.a[L_N];
  e.seq_hi = ll_seq(c.iteration, d.a[L_NAR], d.a[L_ARIDX]) << 16;
  return e;
}

__device__ __forceinline__ void linear_emit(const Ctx &c, const EmitArgs &e, int b, int col, float v, float u, float resv) {
  if (e.epi == EPI_PUSH_LL) {
    // one 32-bit word per element: bf16 partial sum in the low half, sequence number in the high half
    const size_t off = e.push_off + (size_t)b * e.push_n + col;
    const __nv_bfloat16 hv = __float2bfloat16_rn(v);
    const uint32_t word = (uint32_t)(*reinterpret_cast<const unsigned short *>(&hv)) | e.seq_hi;
    for (int peer = 0; peer < e.world; ++peer)
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<uint32_t *>(c.P.peer_inbox[peer]) + off),
                   "r"(word)
                   : "memory");
  } else if (e.epi == EPI_PUSH_F32) {
    const size_t off = e.push_off + (size_t)b * e.push_n + col;
    for (int peer = 0; peer < e.world; ++peer) c.P.peer_inbox[peer][off] = v;
  } else if (e.epi == EPI_SILU_PAIR) {
    // rows come as [gate, gate, up, up]: the threads on gate rows finish the pair (u = the value two rows on)
    if ((col & 2) == 0) {
      const float a = round_bf16(silu_f(round_bf16(v)));
      e.out[(size_t)b * e.ldo + ((col >> 2) << 1) + (col & 1)] = __float2bfloat16_rn(a * round_bf16(u));
    }
  } else {
    e.out[(size_t)b * e.ldo + col] = __float2bfloat16_rn(v + resv);   // resv: the residual element, or 0
  }
}

__device__ void run_linear_tc(const Ctx &c, const TaskDesc &d, LinearState &ls, int task, const uint4 (&gpre)[2], bool ok) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int B = ok ? min(active_tokens(P), kMaxLinearTokens) : 0;
  const int NP = P.tc_tokens;                               // token rows of the operand tile / columns per accumulator
  const int Nmma = min(NP, max(16, (B + 15) & ~15));        // N of the instruction
  const int n0 = d.a[L_N0], rows = d.a[L_N1] - n0, K = d.a[L_K], KT = d.a[L_KT], RB = d.a[L_ROWS];
  const int nkb = d.a[L_KC] / kTcKBlock, kbt = KT / kTcKBlock;
  const int tiles = (rows + RB - 1) / RB;
  const int NST = P.num_stages;
  const uint32_t idesc = umma_idesc(1u, 128, Nmma);
  const bool prof = P.profiler != nullptr && (uint64_t)(task + 1) * 8 <= P.profiler_entries;
  // Several warps issue MMAs concurrently, and MMAs of different threads execute in no fixed order: were they to
  // share an accumulator, the order of the fp32 additions -- and with it the last bit of the result -- would change
  // from launch to launch.  So every issuing warp owns a SET of accumulators (set i, tile t at columns
  // (i * tiles + t) * NP), filled only by its own MMAs, which execute in issue order; the epilogue adds the sets in
  // set order.  As many issuers as the accumulator columns allow, eight at most.  Every MMA accumulates, so the
  // columns start at zero: warps 0-3 clear their lane quadrants.
  const int sets = max(1, min(8, kTcAccCols / (tiles * NP)));
  tc_fence_after_sync();
  if (ok && warp < 4) {
    const uint32_t t0 = c.tmem_base + ((uint32_t)(warp * 32) << 16);
    for (int col = 0; col < sets * tiles * NP; col += 16) tmem_st_zero_x16(t0 + (uint32_t)col);
    tmem_st_wait();
  }
  tc_fence_before_sync();
  // descriptor templates: shared-memory addresses enter as (address >> 4) in the low 14 bits
  const uint64_t desc_hi = umma_desc_k_sw128(0);
  const uint32_t x_base = smem_u32(c.s.xtile) >> 4;
  for (int kt = 0; kt < K; kt += KT) {
    if (ok && !((d.flags & TF_SAME_X_AS_PREV) && KT == K)) {
      stage_x<2>(c, d, B, kt, KT, gpre);   // (a barrier of the compute warps precedes every return)
      fence_proxy_async_smem();            // the tile was written with generic stores; the MMA reads it through the async proxy
    }
    consumer_sync();
    tc_fence_after_sync();
    if (tid == 0 && prof && kt == 0) P.profiler[(size_t)task * 8 + 4] = globaltimer_ns();
    // Ring slots in stream order (row tile, then k blocks).  A slot holds nkb k blocks = 4 nkb MMAs of K = 16; warp w
    // issues MMAs w, w + 8, ... of the slot from its lane 0 and then commits to the slot's empty barrier, which
    // counts eight arrivals: the slot returns to the streaming warp when the MMAs of all warps have read it.
    for (int tile = 0; tile < tiles; ++tile) {
      const uint32_t d_tmem = c.tmem_base + (uint32_t)((warp * tiles + tile) * NP);   // (used by warps < sets only)
      for (int kb = 0; kb < kbt; kb += nkb) {
        const int s = ls.stage;
        const uint32_t ph = ls.phase;
        if (++ls.stage == NST) { ls.stage = 0; ls.phase ^= 1u; }
        if (ok) ok = wait_mbar(c, &c.s.full[s], ph, task);
        if (ok && lane == 0) {
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(c.s.stages + (size_t)s * P.stage_bytes) >> 4;
          for (int m = warp; warp < sets && m < nkb * 4; m += sets) {
            const int j = m >> 2, ks = m & 3;
            const uint32_t a_lo = a_base + (uint32_t)(j * RB * 8 + ks * 2);
            const uint32_t b_lo = x_base + (uint32_t)((kb + j) * NP * 8 + ks * 2);
            umma_bf16_acc(d_tmem, desc_hi | a_lo, desc_hi | b_lo, idesc);
          }
          umma_commit(&c.s.empty[s]);
        }
        __syncwarp();
      }
    }
    // accumulators complete for this k tile / activation tile free again: one arrival per warp
    if (lane == 0) umma_commit(c.s.acc_bar);
    if (!wait_mbar(c, c.s.acc_bar, ls.acc_phase, task)) ok = false;
    ls.acc_phase ^= 1u;
    if (!ok) c.s.flags[0] = 1;
    consumer_sync();
    ok = ok && (c.s.flags[0] == 0);
    if (!ok) break;
  }
  if (tid == 0 && prof) P.profiler[(size_t)task * 8 + 5] = globaltimer_ns();
  if (!ok) { c.s.flags[0] = 1; return; }
  tc_fence_after_sync();
  if (B > 0) {
    const int quad = warp & 3, half = warp >> 2;
    const int nh = Nmma >> 1;   // a multiple of 8
    const EmitArgs ea = emit_args(c, d);
    const int epi = ea.epi;
    const __nv_bfloat16 *resp = reinterpret_cast<const __nv_bfloat16 *>(d.p[3]);
    const int ldr = d.a[L_LDR];
    for (int tile = 0; tile < tiles; ++tile) {
      if (quad * 32 >= RB) break;                           // this warp's lanes hold no row of a tile (warp-uniform)
      const int r_in_tile = quad * 32 + lane;
      const int row = tile * RB + r_in_tile;
      const bool row_ok = r_in_tile < RB && row < rows;
      const uint32_t taddr = c.tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(tile * NP + half * nh);
      for (int c0 = 0; c0 < nh; c0 += 8) {
        uint32_t r[8];
        tmem_ld_x8(taddr + (uint32_t)c0, r);
        for (int st = 1; st < sets; ++st) {   // the other issuers' accumulators of this tile, in set order
          uint32_t r2[8];
          tmem_ld_wait();
          tmem_ld_x8(taddr + (uint32_t)(st * tiles * NP + c0), r2);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
        }
        // residual values of the group's eight tokens: all loads in flight together, ahead of the stores (which the
        // compiler may not move them across: the output may alias the residual)
        float resv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int b = half * nh + c0 + j;
          resv[j] = 0.f;
          if (epi == EPI_RESIDUAL && row_ok && b < B)
            resv[j] = bf16_to_f(__ldcg(resp + (size_t)b * ldr + n0 + row));
        }
        tmem_ld_wait();
        if (tid == 0 && prof && tile == 0 && c0 == 0) P.profiler[(size_t)task * 8 + 6] = globaltimer_ns();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float v = __uint_as_float(r[j]);
          const float u = (epi == EPI_SILU_PAIR) ? __shfl_down_sync(0xffffffffu, v, 2) : 0.f;
          const int b = half * nh + c0 + j;
          if (row_ok && b < B) linear_emit(c, ea, b, n0 + row, v, u, resv[j]);
        }
        if (tid == 0 && prof && tile == 0 && c0 == 0) P.profiler[(size_t)task * 8 + 7] = globaltimer_ns();
      }
    }
  }
  tc_fence_before_sync();   // the accumulators have been read: the next task's MMAs may overwrite them after the task barrier
}

// ---------------------------------------------------------------------------
// FP8 TASK_LINEAR on the tensor path: tcgen05.mma kind::mxf8f6f4 with block scaling, the form the reference uses
// (include/mirage/persistent_kernel/tasks/blackwell/linear_fp8_1d2d_sm100.cuh:69-727).  Geometry as in run_linear_tc
// with one byte per element: a 128-byte k block is 128 columns = one scale group = four MMAs of K = 32.  The scale
// tensors hold four UE8M0 exponents per uint32 (four consecutive groups, 512 columns): such a word per row IS the
// tensor-memory scale column the instruction wants, the group within it is the instruction's scale id.  Per 512
// columns and row tile, 128 weight-scale words (and 128 activation-scale words per 512 columns) are staged in shared
// memory in the [32 lanes][4 words] order tcgen05.cp copies to tensor memory.  A 512-column "super group" of a tile
// belongs to one warp, which copies its scale words into its own eight tensor-memory columns and then issues the 16
// MMAs in order behind the copy; super groups rotate over the issuing warps.
// ---------------------------------------------------------------------------
__device__ void run_linear_fp8_tc(const Ctx &c, const TaskDesc &d, LinearState &ls, int task, bool ok) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int B = ok ? min(active_tokens(P), kMaxLinearTokens) : 0;
  const int NP = P.tc_tokens;
  const int Nmma = min(NP, max(16, (B + 15) & ~15));
  const int n0 = d.a[L_N0], rows = d.a[L_N1] - n0, K = d.a[L_K], KT = d.a[L_KT], RB = d.a[L_ROWS];
  const int nkb = d.a[L_KC] / 128, kbt = KT / 128, nsg = KT / 512;
  const int tiles = (rows + RB - 1) / RB;
  const int NST = P.num_stages;
  uint8_t *xt = c.s.xtile;                                   // [kbt][NP][128 bytes], swizzled
  uint32_t *sfb = reinterpret_cast<uint32_t *>(xt + (size_t)NP * KT);              // [nsg][128 words]
  uint32_t *sfa = sfb + (size_t)nsg * 128;                   // [tiles][nsg][128 words]
  // one accumulator set per issuing warp, added in set order by the epilogue (see run_linear_tc): bit-reproducible
  const int sets = max(1, min(8, kTcAccCols / (tiles * NP)));
  tc_fence_after_sync();
  if (ok && warp < 4) {
    const uint32_t t0 = c.tmem_base + ((uint32_t)(warp * 32) << 16);
    for (int col = 0; col < sets * tiles * NP; col += 16) tmem_st_zero_x16(t0 + (uint32_t)col);
    tmem_st_wait();
  }
  tc_fence_before_sync();
  const uint64_t desc_hi = umma_desc_k_sw128(0);
  const uint32_t x_base = smem_u32(xt) >> 4;
  const uint32_t my_sfa = c.tmem_base + (uint32_t)(kTcAccCols + warp * 8), my_sfb = my_sfa + 4u;
  const uint32_t *ws = reinterpret_cast<const uint32_t *>(d.p[6]);
  const uint32_t *xs = reinterpret_cast<const uint32_t *>(d.p[7]);
  int sg_seq = 0;                                            // running count of (tile, super group) units: owner = sg_seq % 8
  for (int kt = 0; kt < K; kt += KT) {
    if (ok) {
      const bool with_x = !((d.flags & TF_SAME_X_AS_PREV) && KT == K);
      if (with_x) {
        const uint8_t *x = reinterpret_cast<const uint8_t *>(d.p[1]);
        const int ldx = d.a[L_LDX], vecs = KT / 16;
        for (int b = 0; b < B; ++b)
          for (int v = tid; v < vecs; v += kConsumerThreads)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(x_vec<2>(xt, b, v, 0, NP))),
                         "l"(reinterpret_cast<const uint4 *>(x + (size_t)b * ldx + kt) + v)
                         : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
        // activation scale words, token b of super group sg -> word (b % 32) * 4 + b / 32 of the group's block
        const int s0 = d.a[L_XS_S0], s1 = d.a[L_XS_S1];
        // (four loads in flight per thread before the first store: a store to shared memory through a generic
        // pointer keeps the compiler from moving the next load above it)
        for (int i0 = tid; i0 < nsg * 128; i0 += 4 * kConsumerThreads) {
          uint32_t w[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * kConsumerThreads, sg = i >> 7, b = i & 127;
            w[u] = (i < nsg * 128 && b < B) ? __ldcg(xs + (size_t)b * s0 + (size_t)(kt / 512 + sg) * s1) : 0u;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * kConsumerThreads, sg = i >> 7, b = i & 127;
            if (i < nsg * 128) sfb[sg * 128 + (b & 31) * 4 + (b >> 5)] = w[u];
          }
        }
      }
      {
        const int s0 = d.a[L_WS_S0], s1 = d.a[L_WS_S1];
        for (int i0 = tid; i0 < tiles * nsg * 128; i0 += 4 * kConsumerThreads) {
          uint32_t w[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * kConsumerThreads, r = i & 127, uu = i >> 7, tile = uu / nsg, sg = uu - tile * nsg;
            const int row = tile * RB + r;
            w[u] = (i < tiles * nsg * 128 && r < RB && row < rows)
                       ? __ldcg(ws + (size_t)(n0 + row) * s0 + (size_t)(kt / 512 + sg) * s1) : 0u;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * kConsumerThreads, r = i & 127, uu = i >> 7;
            if (i < tiles * nsg * 128) sfa[uu * 128 + (r & 31) * 4 + (r >> 5)] = w[u];
          }
        }
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      fence_proxy_async_smem();
    }
    consumer_sync();
    tc_fence_after_sync();
    for (int tile = 0; tile < tiles; ++tile) {
      const uint32_t d_tmem = c.tmem_base + (uint32_t)((warp * tiles + tile) * NP);   // (used by warps < sets only)
      for (int kb = 0; kb < kbt; kb += nkb) {
        const int s = ls.stage;
        const uint32_t ph = ls.phase;
        if (++ls.stage == NST) { ls.stage = 0; ls.phase ^= 1u; }
        if (ok) ok = wait_mbar(c, &c.s.full[s], ph, task);
        if (ok && lane == 0) {
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(c.s.stages + (size_t)s * P.stage_bytes) >> 4;
          for (int j = 0; j < nkb; ++j) {
            const int g = kb + j, sg = g >> 2;                // k block (= scale group) and its super group within the k tile
            if ((sg_seq + sg) % sets != warp) continue;
            if ((g & 3) == 0 || j == 0) {
              // (first block of the super group that this slot brings: if the group began in an earlier slot the
              // words are already in place, and copying them again behind the earlier MMAs is harmless)
              utccp_sf_128(my_sfa, smem_u32(sfa + (size_t)(tile * nsg + sg) * 128));
              utccp_sf_128(my_sfb, smem_u32(sfb + (size_t)sg * 128));
            }
            const uint32_t idesc = umma_idesc_mxf8(128, Nmma, (uint32_t)(g & 3));
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              umma_mxf8_acc(d_tmem, desc_hi | (a_base + (uint32_t)(j * RB * 8 + ks * 2)),
                            desc_hi | (x_base + (uint32_t)(g * NP * 8 + ks * 2)), idesc, my_sfa, my_sfb);
          }
          umma_commit(&c.s.empty[s]);
        }
        __syncwarp();
      }
      sg_seq += nsg;
    }
    if (lane == 0) umma_commit(c.s.acc_bar);
    if (!wait_mbar(c, c.s.acc_bar, ls.acc_phase, task)) ok = false;
    ls.acc_phase ^= 1u;
    if (!ok) c.s.flags[0] = 1;
    consumer_sync();
    ok = ok && (c.s.flags[0] == 0);
    if (!ok) break;
  }
  if (!ok) { c.s.flags[0] = 1; return; }
  tc_fence_after_sync();
  if (B > 0) {
    const int quad = warp & 3, half = warp >> 2;
    const int nh = Nmma >> 1;
    const EmitArgs ea = emit_args(c, d);
    const __nv_bfloat16 *resp = reinterpret_cast<const __nv_bfloat16 *>(d.p[3]);
    const int ldr = d.a[L_LDR];
    for (int tile = 0; tile < tiles; ++tile) {
      if (quad * 32 >= RB) break;
      const int r_in_tile = quad * 32 + lane;
      const int row = tile * RB + r_in_tile;
      const bool row_ok = r_in_tile < RB && row < rows;
      const uint32_t taddr = c.tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(tile * NP + half * nh);
      for (int c0 = 0; c0 < nh; c0 += 8) {
        uint32_t r[8];
        tmem_ld_x8(taddr + (uint32_t)c0, r);
        for (int st = 1; st < sets; ++st) {
          uint32_t r2[8];
          tmem_ld_wait();
          tmem_ld_x8(taddr + (uint32_t)(st * tiles * NP + c0), r2);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
        }
        float resv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int b = half * nh + c0 + j;
          resv[j] = 0.f;
          if (ea.epi == EPI_RESIDUAL && row_ok && b < B) resv[j] = bf16_to_f(__ldcg(resp + (size_t)b * ldr + n0 + row));
        }
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int b = half * nh + c0 + j;
          if (row_ok && b < B) linear_emit(c, ea, b, n0 + row, __uint_as_float(r[j]), 0.f, resv[j]);
        }
      }
    }
  }
  tc_fence_before_sync();
}

// ---------------------------------------------------------------------------
// FP8 linear: e4m3 weights and activations with one UE8M0 (power-of-two) scale per 128 columns of every
// row, on mma.sync m16n8k32.  Replaces linear_fp8_1d2d_sm100 and its residual form
// (include/mirage/persistent_kernel/tasks/blackwell/linear_fp8_1d2d_sm100.cuh).  The streaming geometry
// is that of the bf16 task with one byte per element: an e4m3 k step of 32 columns spans the same 32 bytes
// of a row as a bf16 step of 16, so the fragment addressing is identical.  Each warp takes whole 128-column
// groups: four mma into a fresh accumulator, then acc += tmp * 2^(ew + ea - 254).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mma_e4m3_16832(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The same contraction with the e4m3 operands widened to f16 in registers (exact: every e4m3 value is an f16 value)
// and two f16 MMAs of k = 16: thread (g, q) holds bytes 4q .. 4q + 3 of a row in each e4m3 fragment register; the
// first two become the f16 fragment's columns (2q, 2q + 1), the last two its columns (2q + 8, 2q + 9), in A and B
// alike, so that both operands see the same permutation of k within the step.
__device__ __forceinline__ void cvt_e4m3x4_f16x4(uint32_t src, uint32_t &lo, uint32_t &hi) {
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
      : "=r"(lo), "=r"(hi)
      : "r"(src));
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_e4m3_as_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  uint32_t al[4], ah[4], bl[2], bh[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) cvt_e4m3x4_f16x4(a[i], al[i], ah[i]);
  cvt_e4m3x4_f16x4(b0, bl[0], bh[0]);
  cvt_e4m3x4_f16x4(b1, bl[1], bh[1]);
  mma_f16_16816(d, al[0], al[1], ah[0], ah[1], bl[0], bh[0]);   // k 0 .. 15 of the step
  mma_f16_16816(d, al[2], al[3], ah[2], ah[3], bl[1], bh[1]);   // k 16 .. 31
}

// 2^(ew - 127) * 2^(ea - 127) as a float, clamped to the normal range
__device__ __forceinline__ float ue8m0_pair_scale(uint32_t ew, uint32_t ea) {
  int e = (int)ew + (int)ea - 127;
  e = max(1, min(254, e));
  return __int_as_float(e << 23);
}

__device__ __forceinline__ uint32_t align16u(uint32_t v) { return (v + 15u) & ~15u; }

// Stage, for k range [k0, k0 + KT): the activation rows and their scale exponents (unless the previous task
// left them in place), and the scale exponents of this task's weight rows.
__device__ void stage_fp8(const Ctx &c, const TaskDesc &d, int B, int k0, int KT, bool with_x) {
  const int tid = threadIdx.x;
  const uint32_t xstride = (uint32_t)KT + kRowPadBytes;
  const int NG = KT / 128, g0 = k0 / 128;
  uint8_t *xt = c.s.xtile;
  uint8_t *xsc = xt + align16u((uint32_t)B * xstride);
  uint8_t *wsc = xsc + align16u((uint32_t)(B * NG));
  if (with_x) {
    const uint8_t *x = reinterpret_cast<const uint8_t *>(d.p[1]);
    const int ldx = d.a[L_LDX];
    const int vecs = KT / 16;
    for (int i = tid; i < B * vecs; i += kConsumerThreads) {   // asynchronous copies, all in flight together
      const int b = i / vecs, v = i - b * vecs;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(xt + (size_t)b * xstride + (size_t)v * 16)),
                   "l"(reinterpret_cast<const uint4 *>(x + (size_t)b * ldx + k0) + v)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    const uint32_t *xs = reinterpret_cast<const uint32_t *>(d.p[7]);
    const int s0 = d.a[L_XS_S0], s1 = d.a[L_XS_S1];
    for (int i = tid; i < B * NG; i += kConsumerThreads) {
      const int b = i / NG, ga = g0 + (i - b * NG);
      const uint32_t word = __ldcg(xs + (size_t)b * s0 + (size_t)(ga >> 2) * s1);
      xsc[i] = (uint8_t)((word >> ((ga & 3) * 8)) & 0xffu);
    }
  }
  {
    const uint32_t *ws = reinterpret_cast<const uint32_t *>(d.p[6]);
    const int s0 = d.a[L_WS_S0], s1 = d.a[L_WS_S1];
    const int n0 = d.a[L_N0], rows = d.a[L_N1] - n0;
    for (int i = tid; i < rows * NG; i += kConsumerThreads) {
      const int r = i / NG, ga = g0 + (i - r * NG);
      const uint32_t word = __ldcg(ws + (size_t)(n0 + r) * s0 + (size_t)(ga >> 2) * s1);
      wsc[i] = (uint8_t)((word >> ((ga & 3) * 8)) & 0xffu);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  consumer_sync();
}

__device__ __forceinline__ void run_linear_fp8(const Ctx &c, const TaskDesc &d, LinearState &ls, int task, bool ok) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int stage = ls.stage;
  uint32_t phase = ls.phase;
  const int B = ok ? min(active_tokens(P), kMaxLinearTokens) : 0;
  const int NT = B <= 8 ? 1 : (B <= 16 ? 2 : (B <= 32 ? 4 : 8));
  const int nt = warp % NT, ks = warp / NT, kstride = 8 / NT;
  const int n0 = d.a[L_N0], n1 = d.a[L_N1], K = d.a[L_K];
  const int KT = d.a[L_KT], KC = d.a[L_KC], R = d.a[L_ROWS];
  const int NST = P.num_stages;
  const int ngc = KC / 128, NG = KT / 128;
  const uint32_t row_stride = (uint32_t)KC + kRowPadBytes;
  const uint32_t xstride = (uint32_t)KT + kRowPadBytes;
  const int g = lane >> 2, q = lane & 3;
  const bool tok_valid = nt * 8 + g < B;
  const bool multi_tile = KT < K;
  const uint32_t a_lane_off = (uint32_t)(lane & 15) * row_stride + (uint32_t)(lane >> 4) * 16u;
  const uint32_t x_lane_base = smem_u32(c.s.xtile) + (uint32_t)(tok_valid ? nt * 8 + g : 0) * xstride + (uint32_t)q * 4u;
  const uint8_t *xsc = c.s.xtile + align16u((uint32_t)B * xstride);
  const uint8_t *wsc = xsc + align16u((uint32_t)(B * NG));
  const uint8_t *xsc0 = xsc + (size_t)(nt * 8 + 2 * q) * NG, *xsc1 = xsc0 + NG;
  int group_seq = 0;
  for (int kt = 0; kt < K; kt += KT) {
    if (B > 0) {
      if (kt > 0) consumer_sync();
      stage_fp8(c, d, B, kt, KT, !((d.flags & TF_SAME_X_AS_PREV) && !multi_tile));
    }
    int gi = 0;
    for (int r0 = n0; r0 < n1; r0 += R, ++gi) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const uint8_t *wsc0 = wsc + (size_t)(r0 - n0 + g) * NG, *wsc1 = wsc0 + 8 * NG;
      for (int kc = 0; kc < KT; kc += KC) {
        const int s = stage;
        const uint32_t ph = phase;
        if (++stage == NST) { stage = 0; phase ^= 1u; }
        if (ok) ok = wait_mbar(c, &c.s.full[s], ph, task);
        if (ok && B > 0) {
          const uint32_t a_base = smem_u32(c.s.stages + (size_t)s * P.stage_bytes) + a_lane_off;
          const uint32_t x_base = x_lane_base + (uint32_t)kc;
          for (int m = ks; m < ngc; m += kstride) {
            uint32_t a[4][4], b[4][2];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const uint32_t o = (uint32_t)(m * 4 + u) * 32u;
              ldmatrix_x4(a[u], a_base + o);
              asm volatile("ld.shared.b32 %0, [%1];" : "=r"(b[u][0]) : "r"(x_base + o));
              asm volatile("ld.shared.b32 %0, [%1];" : "=r"(b[u][1]) : "r"(x_base + o + 16u));
            }
            float t0[4] = {0.f, 0.f, 0.f, 0.f}, t1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (!tok_valid) b[u][0] = b[u][1] = 0u;
              if (u & 1) mma_e4m3_16832(t1, a[u], b[u][0], b[u][1]);
              else mma_e4m3_16832(t0, a[u], b[u][0], b[u][1]);
            }
            const int gt = kc / 128 + m;
            const uint32_t ew0 = wsc0[gt], ew1 = wsc1[gt], ea0 = xsc0[gt], ea1 = xsc1[gt];
            acc[0] += (t0[0] + t1[0]) * ue8m0_pair_scale(ew0, ea0);
            acc[1] += (t0[1] + t1[1]) * ue8m0_pair_scale(ew0, ea1);
            acc[2] += (t0[2] + t1[2]) * ue8m0_pair_scale(ew1, ea0);
            acc[3] += (t0[3] + t1[3]) * ue8m0_pair_scale(ew1, ea1);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&c.s.empty[s]);
      }
      if (B > 0) {
        float *part = c.s.partial + (size_t)((multi_tile ? gi : group_seq) & 1) * (8 * 16 * 8);
        float *mine = part + (size_t)warp * (16 * 8);
        float2 *p0 = reinterpret_cast<float2 *>(mine + g * 8 + q * 2);
        float2 *p1 = reinterpret_cast<float2 *>(mine + (g + 8) * 8 + q * 2);
        if (multi_tile && kt > 0) {
          float2 o0 = *p0, o1 = *p1;
          *p0 = make_float2(o0.x + acc[0], o0.y + acc[1]);
          *p1 = make_float2(o1.x + acc[2], o1.y + acc[3]);
        } else {
          *p0 = make_float2(acc[0], acc[1]);
          *p1 = make_float2(acc[2], acc[3]);
        }
        if (!multi_tile) {
          consumer_sync();
          linear_group_epilogue<true>(c, d, B, NT, r0, min(R, n1 - r0), part);
        }
      }
      ++group_seq;
    }
  }
  if (!ok) c.s.flags[0] = 1;
  if (B > 0 && multi_tile) {
    consumer_sync();
    int gi = 0;
    for (int r0 = n0; r0 < n1; r0 += R, ++gi)
      linear_group_epilogue<true>(c, d, B, NT, r0, min(R, n1 - r0), c.s.partial + (size_t)(gi & 1) * (8 * 16 * 8));
  }
  ls.stage = stage;
  ls.phase = phase;
}

// TASK_QUANTIZE_FP8: bf16 -> e4m3 with one scale per (row, 128 columns); a warp owns a pack of four groups.
// Follows per_token_group_quantize_fp8 (include/mirage/persistent_kernel/tasks/blackwell/
// per_token_group_quantize_fp8.cuh:33-160): amax clamped at 1e-10, scale = amax / 448, for UE8M0 rounded up
// to a power of two (computed on the exponent bits, which is exact) and packed four to a uint32 word.
__device__ void run_quantize_fp8(const Ctx &c, const TaskDesc &d) {
  const KernelParams &P = c.P;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = d.a[2], ldx = d.a[3], ldq = d.a[4], per_tok = d.a[6], s0 = d.a[7], s1 = d.a[8], pk = d.a[9];
  const bool ue8m0 = d.a[5] != 0;
  const int ng = K / 128;
  const int active = active_tokens(P);
  const __nv_bfloat16 *x = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  uint8_t *qo = reinterpret_cast<uint8_t *>(d.p[1]);
  for (int u = d.a[0] + warp; u < d.a[1]; u += kConsumerThreads / 32) {
    const int row = u / pk, j = u - row * pk;
    if (row / per_tok >= active) continue;
    uint32_t word = 0;
    for (int gi = 0; gi < 4; ++gi) {
      const int gidx = j * 4 + gi;
      if (gidx >= ng) break;
      const uint2 raw = __ldcg(reinterpret_cast<const uint2 *>(x + (size_t)row * ldx + (size_t)gidx * 128) + lane);
      float v[4];
      v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xffff0000u);
      v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xffff0000u);
      float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      amax = fmaxf(amax, 1e-10f);
      float scale = __fdiv_rn(amax, 448.0f);
      if (ue8m0) {
        const uint32_t bits = __float_as_uint(scale);
        uint32_t e = (bits >> 23) & 0xffu;
        if (bits & 0x7fffffu) ++e;                 // ceil(log2(scale)) + 127
        e = min(e, 254u);
        scale = __uint_as_float(e << 23);
        word |= e << (8 * gi);
      } else if (lane == 0) {
        reinterpret_cast<float *>(d.p[2])[(size_t)row * s0 + (size_t)gidx * s1] = scale;
      }
      float qv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = fminf(fmaxf(__fdiv_rn(v[i], scale), -448.0f), 448.0f);
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(qv[0], qv[1]), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(qv[2], qv[3]), __NV_SATFINITE, __NV_E4M3);
      *reinterpret_cast<uint32_t *>(qo + (size_t)row * ldq + (size_t)gidx * 128 + (size_t)lane * 4) = lo | (hi << 16);
    }
    if (ue8m0 && lane == 0) reinterpret_cast<uint32_t *>(d.p[2])[(size_t)row * s0 + (size_t)j * s1] = word;
  }
}

// ---------------------------------------------------------------------------
// Mixture of experts (general instantiation only)
// ---------------------------------------------------------------------------
// TASK_MOE_ROUTING: DeepSeek-V3 group-aware sigmoid routing, one warp per token
// (include/mirage/persistent_kernel/tasks/blackwell/topk_sigmoid_sm100.cuh:75-362): selection on
// sigmoid + bias, group score = sum of the group's two largest biased scores, `keep` groups survive (ties: lowest
// group), top-k experts by repeated argmax (ties: lowest expert), weights from the unbiased scores.  The list of
// active experts is written in ascending order (the reference's order depends on atomics).  The logits are
// zeroed after they are read, as the reference does for its accumulating gate projection.
__device__ void run_moe_routing(const Ctx &c, const TaskDesc &d) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int E = d.a[0], topk = d.a[1], groups = d.a[2], keep = d.a[3];
  const float scaling = __int_as_float(d.a[4]);
  const int ldl = d.a[5], ldw = d.a[6], ldr = d.a[7];
  const bool f32_in = d.a[8] != 0;
  // expert parallelism: this rank runs experts [e_lo, e_hi) only.  Selection and normalisation are those of the whole
  // expert set (every rank computes the same routing); slots of experts of other ranks get weight 0 and stay out
  // of the active list, so the grouped projections skip them and the weighted sum ignores their rows.
  const int e_lo = d.a[9], e_hi = d.a[10];
  const int per = E / groups;
  const int B = min(active_tokens(P), ldr);
  float *wout = reinterpret_cast<float *>(d.p[2]);
  int *routing = reinterpret_cast<int *>(d.p[3]);
  int *active = reinterpret_cast<int *>(d.p[4]);
  const float *bias = reinterpret_cast<const float *>(d.p[1]);
  // shared: per warp [E] unbiased, [E] biased, [64] group scores; then [E] marks, [8] warp counts
  float *wbase = reinterpret_cast<float *>(c.s.xtile) + (size_t)warp * (2 * E + 64);
  float *sc = wbase, *bi = wbase + E, *gs = wbase + 2 * E;
  int *mark = reinterpret_cast<int *>(reinterpret_cast<float *>(c.s.xtile) + (size_t)8 * (2 * E + 64));
  int *wcount = mark + E;
  for (int i = tid; i < E * ldr; i += kConsumerThreads) routing[i] = 0;
  for (int i = tid; i < E; i += kConsumerThreads) mark[i] = 0;
  consumer_sync();
  const bool softmax = d.a[11] != 0;   // moe_topk_softmax_routing_layer: scores = softmax over the experts, no bias, logits kept
  for (int row = warp; row < B; row += 8) {
    float row_max = -INFINITY;
    for (int e = lane; e < E; e += 32) {
      float logit;
      if (f32_in) {
        float *lp = reinterpret_cast<float *>(d.p[0]) + (size_t)row * ldl + e;
        logit = __ldcg(lp);
        if (!softmax) *lp = 0.f;
      } else {
        __nv_bfloat16 *lp = reinterpret_cast<__nv_bfloat16 *>(d.p[0]) + (size_t)row * ldl + e;
        logit = bf16_to_f(__ldcg(lp));
        if (!softmax) *lp = __float2bfloat16_rn(0.f);
      }
      if (softmax) {
        sc[e] = logit;
        row_max = fmaxf(row_max, logit);
      } else {
        const float sig = __fdiv_rn(1.0f, 1.0f + expf(-logit));
        sc[e] = sig;
        bi[e] = sig + __ldg(&bias[e]);
      }
    }
    if (softmax) {
      // exp(x - max) / sum in fp32 (tasks/blackwell/topk_softmax_sm100.cuh:193-216); selection on the probabilities
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, o));
      float row_sum = 0.f;
      for (int e = lane; e < E; e += 32) {
        const float p = expf(sc[e] - row_max);
        sc[e] = p;
        row_sum += p;
      }
      row_sum = warp_sum(row_sum);
      const float inv_sum = __fdiv_rn(1.0f, row_sum);
      for (int e = lane; e < E; e += 32) {
        const float p = sc[e] * inv_sum;
        sc[e] = p;
        bi[e] = p;
      }
    }
    __syncwarp();
    for (int g = lane; g < groups; g += 32) {
      float t1 = bi[g * per], t2 = -1e30f;
      for (int i = 1; i < per; ++i) {
        const float v = bi[g * per + i];
        if (v > t1) { t2 = t1; t1 = v; }
        else if (v > t2) t2 = v;
      }
      gs[g] = t1 + t2;
    }
    __syncwarp();
    unsigned long long selected = 0ull;
    for (int k = 0; k < keep; ++k) {
      int best = 0;
      float best_s = -1e30f;
      for (int g = 0; g < groups; ++g)
        if (!((selected >> g) & 1ull) && gs[g] > best_s) { best_s = gs[g]; best = g; }
      selected |= 1ull << best;
    }
    for (int e = lane; e < E; e += 32)
      if (!((selected >> (e / per)) & 1ull)) bi[e] = -10000.f;
    __syncwarp();
    float total = 0.f;
    if (lane < 32 && lane < topk) gs[32 + lane] = 0.f;
    __syncwarp();
    for (int k = 0; k < topk; ++k) {
      float mv = -3.0e38f;
      int me = E;
      for (int e = lane; e < E; e += 32) {
        const float v = bi[e];
        if (v > mv) { mv = v; me = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, mv, o);
        const int oe = __shfl_xor_sync(0xffffffffu, me, o);
        if (ov > mv || (ov == mv && oe < me)) { mv = ov; me = oe; }
      }
      if (lane == 0) {
        const float orig = sc[me];
        wout[(size_t)row * ldw + k] = orig;
        total += orig;
        if (me >= e_lo && me < e_hi) {
          routing[(size_t)me * ldr + row] = k + 1;
          mark[me] = 1;
        } else {
          gs[32 + k] = -1.f;   // (group scores are dead by now: remember that slot k belongs to another rank)
        }
        bi[me] = -10000.f;
      }
      __syncwarp();
    }
    if (lane == 0) {
      const float inv = __fdiv_rn(1.0f, total + 1e-20f);
      for (int k = 0; k < topk; ++k) {
        const bool local = gs[32 + k] >= 0.f;
        wout[(size_t)row * ldw + k] = local ? wout[(size_t)row * ldw + k] * inv * scaling : 0.f;
      }
    }
    __syncwarp();
  }
  consumer_sync();
  // ascending list of the experts that received a token; count at index E, unused entries -1
  int base = 0;
  for (int e0 = 0; e0 < E; e0 += kConsumerThreads) {
    const int e = e0 + tid;
    const bool on = e < E && mark[e] != 0;
    const unsigned bal = __ballot_sync(0xffffffffu, on);
    if (lane == 0) wcount[warp] = __popc(bal);
    consumer_sync();
    int before = base;
    for (int w = 0; w < warp; ++w) before += wcount[w];
    if (on) active[before + __popc(bal & ((1u << lane) - 1u))] = e;
    int all = 0;
    for (int w = 0; w < 8; ++w) all += wcount[w];
    base += all;
    consumer_sync();
  }
  for (int i = base + tid; i < E; i += kConsumerThreads) active[i] = -1;
  if (tid == 0) active[E] = base;
}

// TASK_MOE_GEMM: out[b, slot, n0:n1] = x_row . W[e, n, :] for every active expert e and every token routed to it
// (moe_w13 / moe_w2, bf16 or e4m3 with float32 scales per 128 columns; the scales are floored to powers of two
// by taking their exponent bits, as fp8_group_gemm_sm100.cuh:1378 does).  The task owns the row range [n0, n1) of
// EVERY expert: all workers walk the same active list, so the load is balanced whatever the routing.  The
// streamer walks the same list (it waits for the routing first) and streams the panel of each active expert.
__device__ void run_moe_gemm(const Ctx &c, const TaskDesc &d, LinearState &ls, int task, bool ok) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int stage = ls.stage;
  uint32_t phase = ls.phase;
  const bool fp8 = (d.flags & TF_FP8) != 0;
  const uint32_t esz = fp8 ? 1u : 2u;
  const int Bt = ok ? min(active_tokens(P), kMaxLinearTokens) : 0;
  const int n0 = d.a[L_N0], n1 = d.a[L_N1], K = d.a[L_K], N = d.a[L_N];
  const int KT = d.a[L_KT], KC = d.a[L_KC], R = d.a[L_ROWS];
  const int E = d.a[M_NEXP], topk = d.a[M_NTOPK], ldr = d.a[M_LDR];
  const bool per_slot = d.a[M_PER_SLOT] != 0;
  const int NST = P.num_stages;
  const uint32_t seg = (uint32_t)KC * esz, row_stride = seg + kRowPadBytes;
  const uint32_t xstride = (uint32_t)KT * esz + kRowPadBytes;
  const int NG = fp8 ? KT / 128 : 0, ngtot = K / 128;
  const int g = lane >> 2, q = lane & 3;
  const int nkt = K / KT;
  const bool multi_tile = nkt > 1;
  const int *routing = reinterpret_cast<const int *>(d.p[4]);
  const int *active = reinterpret_cast<const int *>(d.p[5]);
  // token | slot << 8 of an expert's tokens (token < 64, slot < 255): two lists, the expert being computed and the next
  unsigned short *tokmaps = reinterpret_cast<unsigned short *>(c.s.red);
  int *cnt_s = c.s.flags + 8;
  const int n_act = ok ? min(__ldcg(&active[E]), E) : 0;
  const uint32_t a_lane_off = (uint32_t)(lane & 15) * row_stride + (uint32_t)(lane >> 4) * 16u;
  const uint8_t *xg = reinterpret_cast<const uint8_t *>(d.p[1]);
  __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  if (n_act <= 0) {
    if (!ok) c.s.flags[0] = 1;
    return;
  }
  // The loop runs over steps (expert, k tile).  A step's operands -- the gathered activation rows of the expert's
  // tokens, their float32 scales and the scales of this task's weight rows, copied raw (the power-of-two floor is
  // taken from the exponent bits where they are used) -- live in a region of the activation tile: rows, token
  // scales, weight-row scales.  While one step computes, the token list of the next expert is built and the next
  // step's operands are copied asynchronously into the free part of the tile (after the current region, or in front
  // of it), so that a step does not begin with a round trip to global memory; a step whose operands do not fit beside
  // the current ones is staged after it.
  auto region_bytes = [&](int cnt) -> uint32_t {
    const int n = max(cnt, 1);
    return align16u((uint32_t)n * xstride) + 4u * (uint32_t)((n * NG + 3) & ~3) + align16u(4u * (uint32_t)((n1 - n0) * NG));
  };
  // routing entries of one expert, held by warps 0 and 1 (token = warp * 32 + lane)
  auto load_routing = [&](int j) -> int {
    if (warp >= 2 || j >= n_act) return 0;
    const int b = warp * 32 + lane;
    return (b < Bt) ? __ldcg(&routing[(size_t)__ldcg(&active[j]) * ldr + b]) : 0;
  };
  // warps 0 and 1: the expert's tokens in token order -> list `which`, counts -> cnt_s[0..1]
  auto build_tokmap = [&](int r, int which) {
    if (warp < 2) {
      unsigned short *tm = tokmaps + which * 64;
      const int b = warp * 32 + lane;
      const unsigned bal = __ballot_sync(0xffffffffu, r != 0);
      if (lane == 0) cnt_s[warp] = __popc(bal);
      if (warp == 0 && r != 0) tm[__popc(bal & ((1u << lane) - 1u))] = (unsigned short)(b | ((r - 1) << 8));
      asm volatile("bar.sync 2, 64;");   // the second half is appended after the first: it needs that count
      if (warp == 1 && r != 0) tm[cnt_s[0] + __popc(bal & ((1u << lane) - 1u))] = (unsigned short)(b | ((r - 1) << 8));
    }
  };
  // asynchronous copies of one step's operands into the region at `off` (committed, not waited for)
  auto stage_step = [&](int e, int cnt, int which, int kt, uint32_t off) {
    const unsigned short *tm = tokmaps + which * 64;
    uint8_t *xr = c.s.xtile + off;
    float *xsc = reinterpret_cast<float *>(xr + align16u((uint32_t)max(cnt, 1) * xstride));
    float *wsc = xsc + (size_t)((max(cnt, 1) * NG + 3) & ~3);
    const int vecs = (int)((uint32_t)KT * esz / 16u);
    for (int i = tid; i < cnt * vecs; i += kConsumerThreads) {
      const int t = i / vecs, v = i - t * vecs;
      const int tmv = tm[t];
      const size_t xrow = per_slot ? (size_t)(tmv & 0xff) * topk + (tmv >> 8) : (size_t)(tmv & 0xff);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(xr + (size_t)t * xstride + (size_t)v * 16)),
                   "l"(reinterpret_cast<const uint4 *>(xg + (xrow * d.a[L_LDX] + kt) * esz) + v)
                   : "memory");
    }
    if (fp8) {
      const float *xs = reinterpret_cast<const float *>(d.p[7]);
      const float *ws = reinterpret_cast<const float *>(d.p[6]);
      const int g0 = kt / 128;
      if (((NG | ngtot) & 3) == 0) {
        // four scales per copy: a row's scales of this k tile are NG consecutive floats, 16-byte aligned on both sides
        const int nv = NG >> 2;
        for (int i = tid; i < cnt * nv; i += kConsumerThreads) {
          const int t = i / nv, v = i - t * nv;
          const int tmv = tm[t];
          const size_t xrow = per_slot ? (size_t)(tmv & 0xff) * topk + (tmv >> 8) : (size_t)(tmv & 0xff);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(xsc + (size_t)t * NG + v * 4)),
                       "l"(&xs[xrow * ngtot + g0 + v * 4])
                       : "memory");
        }
        for (int i = tid; i < (n1 - n0) * nv; i += kConsumerThreads) {
          const int r = i / nv, v = i - r * nv;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(wsc + (size_t)r * NG + v * 4)),
                       "l"(&ws[((size_t)e * N + n0 + r) * ngtot + g0 + v * 4])
                       : "memory");
        }
      } else {
        for (int i = tid; i < cnt * NG; i += kConsumerThreads) {
          const int t = i / NG, gi = i - t * NG;
          const int tmv = tm[t];
          const size_t xrow = per_slot ? (size_t)(tmv & 0xff) * topk + (tmv >> 8) : (size_t)(tmv & 0xff);
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(xsc + i)), "l"(&xs[xrow * ngtot + g0 + gi]) : "memory");
        }
        for (int i = tid; i < (n1 - n0) * NG; i += kConsumerThreads) {
          const int r = i / NG, gi = i - r * NG;
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(wsc + i)),
                       "l"(&ws[((size_t)e * N + n0 + r) * ngtot + g0 + gi])
                       : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // first step: token list and operands of the first expert, synchronously
  consumer_sync();
  int r_next = load_routing(0);
  build_tokmap(r_next, 0);
  r_next = load_routing(1);
  consumer_sync();
  int cnt = cnt_s[0] + cnt_s[1];
  uint32_t off = 0;
  stage_step(__ldcg(&active[0]), cnt, 0, 0, 0u);
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  consumer_sync();

  for (int j = 0; j < n_act; ++j) {
    const int e = __ldcg(&active[j]);
    const int which = j & 1;
    const unsigned short *tokmap = tokmaps + which * 64;
    const int NT = cnt <= 8 ? 1 : (cnt <= 16 ? 2 : (cnt <= 32 ? 4 : 8));
    const int nt = warp % NT, ks = warp / NT, kstride = 8 / NT;
    const bool tok_valid = nt * 8 + g < cnt;
    for (int kt = 0, kti = 0; kt < K; kt += KT, ++kti) {
      // ---- the next step: token list (new expert) and operand copies ----
      const bool last_tile = kti == nkt - 1;
      const bool has_next = !(last_tile && j == n_act - 1);
      int cnt_n = cnt;
      if (has_next && last_tile) {
        build_tokmap(r_next, which ^ 1);
        r_next = load_routing(j + 2);
        consumer_sync();
        cnt_n = cnt_s[0] + cnt_s[1];
      }
      const int e_n = last_tile ? (has_next ? __ldcg(&active[j + 1]) : e) : e;
      const int which_n = last_tile ? which ^ 1 : which;
      const int kt_n = last_tile ? 0 : kt + KT;
      const uint32_t need_c = region_bytes(cnt), need_n = region_bytes(cnt_n);
      uint32_t off_n = off + need_c;
      bool ahead = has_next;
      if (off_n + need_n > (uint32_t)P.x_tile_bytes) {
        off_n = 0;
        if (need_n > off) ahead = false;
      }
      if (has_next && ahead) stage_step(e_n, cnt_n, which_n, kt_n, off_n);

      // ---- this step ----
      const uint8_t *xr = c.s.xtile + off;
      const float *xsc = reinterpret_cast<const float *>(xr + align16u((uint32_t)max(cnt, 1) * xstride));
      const float *wsc = xsc + (size_t)((max(cnt, 1) * NG + 3) & ~3);
      const float *xsc0 = xsc + (size_t)(nt * 8 + 2 * q) * NG, *xsc1 = xsc0 + NG;
      const uint32_t x_lane_base = smem_u32(xr) + (uint32_t)(tok_valid ? nt * 8 + g : 0) * xstride + (uint32_t)q * 4u;
      int gi = 0;
      for (int r0 = n0; r0 < n1; r0 += R, ++gi) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const float *wsc0 = wsc + (size_t)(r0 - n0 + g) * NG, *wsc1 = wsc0 + 8 * NG;
        for (int kc = 0; kc < KT; kc += KC) {
          const int s = stage;
          const uint32_t ph = phase;
          if (++stage == NST) { stage = 0; phase ^= 1u; }
          if (ok) ok = wait_mbar(c, &c.s.full[s], ph, task);
          if (ok && cnt > 0) {
            const uint32_t a_base = smem_u32(c.s.stages + (size_t)s * P.stage_bytes) + a_lane_off;
            const uint32_t x_base = x_lane_base + (uint32_t)kc * esz;
            const int nquad = (int)(seg / 128u);          // groups of four 32-byte k steps
            for (int m = ks; m < nquad; m += kstride) {
              uint32_t a[4][4], b[4][2];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const uint32_t o = (uint32_t)(m * 4 + u) * 32u;
                ldmatrix_x4(a[u], a_base + o);
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(b[u][0]) : "r"(x_base + o));
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(b[u][1]) : "r"(x_base + o + 16u));
                if (!tok_valid) b[u][0] = b[u][1] = 0u;
              }
              if (fp8) {
                float t0[4] = {0.f, 0.f, 0.f, 0.f}, t1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  if (u & 1) mma_e4m3_as_f16(t1, a[u], b[u][0], b[u][1]);
                  else mma_e4m3_as_f16(t0, a[u], b[u][0], b[u][1]);
                }
                const int gt = kc / 128 + m;
                const uint32_t ew0 = (__float_as_uint(wsc0[gt]) >> 23) & 0xffu, ew1 = (__float_as_uint(wsc1[gt]) >> 23) & 0xffu;
                const uint32_t ea0 = (__float_as_uint(xsc0[gt]) >> 23) & 0xffu, ea1 = (__float_as_uint(xsc1[gt]) >> 23) & 0xffu;
                acc[0] += (t0[0] + t1[0]) * ue8m0_pair_scale(ew0, ea0);
                acc[1] += (t0[1] + t1[1]) * ue8m0_pair_scale(ew0, ea1);
                acc[2] += (t0[2] + t1[2]) * ue8m0_pair_scale(ew1, ea0);
                acc[3] += (t0[3] + t1[3]) * ue8m0_pair_scale(ew1, ea1);
              } else {
#pragma unroll
                for (int u = 0; u < 4; ++u) mma_bf16_16816(acc, a[u], b[u][0], b[u][1]);
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&c.s.empty[s]);
        }
        // partial tiles of the eight warps: two buffers, used by row groups in turn (a task with several k tiles has
        // at most two row groups, whose partials stay there across the tiles)
        float *part = c.s.partial + (size_t)(gi & 1) * (8 * 16 * 8);
        float *mine = part + (size_t)warp * (16 * 8);
        float2 *p0 = reinterpret_cast<float2 *>(mine + g * 8 + q * 2);
        float2 *p1 = reinterpret_cast<float2 *>(mine + (g + 8) * 8 + q * 2);
        if (kti > 0) {
          float2 o0 = *p0, o1 = *p1;
          *p0 = make_float2(o0.x + acc[0], o0.y + acc[1]);
          *p1 = make_float2(o1.x + acc[2], o1.y + acc[3]);
        } else {
          *p0 = make_float2(acc[0], acc[1]);
          *p1 = make_float2(acc[2], acc[3]);
        }
        // after the last k tile: sum the warps' partials and write the rows, for the two row groups held at a time
        const bool pair_done = (gi & 1) == 1 || r0 + R >= n1;
        if (last_tile && pair_done) {
          consumer_sync();
          for (int gg = gi & ~1; gg <= gi; ++gg) {
            const float *pp = c.s.partial + (size_t)(gg & 1) * (8 * 16 * 8);
            const int rbase = n0 + gg * R;
            const int rows = min(R, n1 - rbase);
            for (int item = tid; item < cnt * 16; item += kConsumerThreads) {
              const int t = item >> 4, r = item & 15;
              if (r >= rows) continue;
              float v = 0.f;
              for (int w = t >> 3; w < 8; w += NT) v += pp[(w * 16 + r) * 8 + (t & 7)];
              const int tmv = tokmap[t];
              out[((size_t)(tmv & 0xff) * topk + (tmv >> 8)) * d.a[L_LDO] + rbase + r] = __float2bfloat16_rn(v);
            }
          }
          if (r0 + R < n1) consumer_sync();   // further row groups reuse the buffers
        }
      }
      // ---- hand over to the next step ----
      if (has_next && !ahead) {
        consumer_sync();                     // every warp is done with the current region
        stage_step(e_n, cnt_n, which_n, kt_n, 0u);
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      consumer_sync();
      off = off_n;
      cnt = cnt_n;
    }
  }
  if (!ok) c.s.flags[0] = 1;
  ls.stage = stage;
  ls.phase = phase;
}

// TASK_MOE_SILU_MUL: rows of [gate | up] -> bf16(silu(gate)) * up  (tasks/ampere/silu_mul.cuh:20-42 on the
// flattened [token x slot] rows, as register_moe_silu_mul_task sets it up)
__device__ void run_moe_silu_mul(const Ctx &c, const TaskDesc &d) {
  const int I = d.a[2], ldi = d.a[3], ldo = d.a[4];
  const int r1 = min(d.a[1], active_tokens(c.P) * d.a[5]);
  const __nv_bfloat16 *in = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  for (int r = d.a[0]; r < r1; ++r)
    for (int j = threadIdx.x; j < I; j += kConsumerThreads) {
      const float gv = bf16_to_f(__ldcg(&in[(size_t)r * ldi + j]));
      const float uv = bf16_to_f(__ldcg(&in[(size_t)r * ldi + I + j]));
      const float a = round_bf16(gv / (1.0f + expf(-gv)));
      out[(size_t)r * ldo + j] = __float2bfloat16_rn(a * uv);
    }
}

// TASK_MOE_MUL_SUM_ADD: out[b, h] = residual[b, h] + sum_k in[b, k, h] * w[b, k]  (mul_sum_add_sm100.cuh:19-49)
__device__ void run_moe_mul_sum_add(const Ctx &c, const TaskDesc &d) {
  const int c0 = d.a[0], c1 = d.a[1], H = d.a[2], topk = d.a[3], ldo = d.a[4], ldres = d.a[5], ldw = d.a[6];
  const int B = min(d.a[7], active_tokens(c.P));
  const __nv_bfloat16 *in = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  const float *w = reinterpret_cast<const float *>(d.p[1]);
  const __nv_bfloat16 *res = reinterpret_cast<const __nv_bfloat16 *>(d.p[3]);
  __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  for (int b = 0; b < B; ++b)
    for (int h = c0 + threadIdx.x; h < c1; h += kConsumerThreads) {
      float acc = res ? bf16_to_f(__ldcg(&res[(size_t)b * ldres + h])) : 0.f;
      for (int k = 0; k < topk; ++k) {
        const float wk = __ldcg(&w[(size_t)b * ldw + k]);   // 0: the slot's expert lives on another rank (row never written)
        if (wk != 0.f) acc += bf16_to_f(__ldcg(&in[((size_t)b * topk + k) * H + h])) * wk;
      }
      out[(size_t)b * ldo + h] = __float2bfloat16_rn(acc);
    }
}

// ---------------------------------------------------------------------------
// Multi-head latent attention decode (general instantiation only)
// ---------------------------------------------------------------------------
constexpr int kMlaDk = 576, kMlaDv = 512;
constexpr int kMlaRow = kMlaDk * 2 + 16;      // shared-memory row stride of q / kv rows (bytes, conflict-free ldmatrix)
constexpr int kMlaSub = 64;                   // kv rows per shared-memory tile
constexpr int kMlaSplit = 128;                // kv rows per split
constexpr int kMlaPRow = kMlaSub * 2 + 16;    // row stride of the probability tile

// TASK_MLA_APPEND: the request's new [c_latent | k_pe] rows go to their positions in the paged cache
// (step 1 of mla_kv_cache_gather_sm100.cuh:36-128; the decode tasks read the paged cache in place, so the
// reference's second step -- copying the whole sequence to a contiguous buffer -- has no counterpart).
__device__ void run_mla_append(const Ctx &c, const TaskDesc &d) {
  const KernelParams &P = c.P;
  const int slot = d.a[0], ldc = d.a[1], ldp = d.a[2], page = d.a[3], dk = d.a[4], dv = d.a[5];
  const int q0 = __ldcg(&P.meta.qo_indptr[slot]);
  const int nq = __ldcg(&P.meta.qo_indptr[slot + 1]) - q0;
  const int kv0 = __ldcg(&P.meta.paged_kv_indptr[slot]);
  const int npages = __ldcg(&P.meta.paged_kv_indptr[slot + 1]) - kv0;
  if (nq <= 0 || npages <= 0) return;
  const int seq_len = (npages - 1) * page + __ldcg(&P.meta.paged_kv_last_page_len[slot]);
  const __nv_bfloat16 *lat = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  const __nv_bfloat16 *pe = reinterpret_cast<const __nv_bfloat16 *>(d.p[1]);
  __nv_bfloat16 *cache = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  for (int tok = 0; tok < nq; ++tok) {
    const int pos = seq_len - nq + tok;
    if (pos < 0) continue;
    const int pid = __ldcg(&P.meta.paged_kv_indices[kv0 + pos / page]);
    __nv_bfloat16 *dst = cache + ((size_t)pid * page + pos % page) * dk;
    for (int v = threadIdx.x; v < dk / 8; v += kConsumerThreads) {
      const uint4 val = v < dv / 8 ? __ldcg(reinterpret_cast<const uint4 *>(lat + (size_t)(q0 + tok) * ldc) + v)
                                   : __ldcg(reinterpret_cast<const uint4 *>(pe + (size_t)(q0 + tok) * ldp) + (v - dv / 8));
      reinterpret_cast<uint4 *>(dst)[v] = val;
    }
  }
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}

// TASK_MLA_DECODE: one query token x one 128-row split of its kv range x 16 heads, on mma.sync m16n8k16
// (replaces mla_mtp_decode_sm100 and its tensor-parallel variants).  Per 64-row tile: warp w computes the scores
// of kv rows [8w, 8w + 8) for all 16 heads (36 k steps over the 576 latent + rope dims), the row maxima and sums
// go through shared memory, the probabilities are written as a bf16 tile, and warp w accumulates output columns
// [64w, 64w + 64) of P.V with V read transposed from the same kv tile.  Output: O normalised by the split's own
// sum (bf16) and the split's log-sum-exp (fp32); TASK_MLA_REDUCE merges the splits.
__device__ void run_mla_decode(const Ctx &c, const TaskDesc &d) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q = lane & 3;
  const int t = d.a[0], split = d.a[1], head0 = d.a[2], H = d.a[3], S = d.a[4], page = d.a[5], ldq = d.a[6];
  const float scale = __int_as_float(d.a[7]);
  if (t >= active_tokens(P)) return;
  // the request that owns token t, its length and the number of kv positions the token may see
  int kv0 = 0, lim = 0;
  size_t contiguous_base = 0;
  if (page > 0) {
    // every thread tests one request slot; the owner publishes its index
    int *owner = c.s.flags + 10;
    if (tid == 0) *owner = -1;
    consumer_sync();
    for (int r = tid; r < P.max_num_batched_requests; r += kConsumerThreads) {
      const int a0 = __ldcg(&P.meta.qo_indptr[r]), a1 = __ldcg(&P.meta.qo_indptr[r + 1]);
      if (t >= a0 && t < a1) *owner = r;
    }
    consumer_sync();
    const int r = *owner;
    if (r >= 0) {
      const int q0 = __ldcg(&P.meta.qo_indptr[r]), q1 = __ldcg(&P.meta.qo_indptr[r + 1]);
      kv0 = __ldcg(&P.meta.paged_kv_indptr[r]);
      const int npages = __ldcg(&P.meta.paged_kv_indptr[r + 1]) - kv0;
      const int seq_len = (npages - 1) * page + __ldcg(&P.meta.paged_kv_last_page_len[r]);
      lim = seq_len - (q1 - q0) + (t - q0) + 1;
    }
  } else {
    const int q_len = d.a[8], kv_len = d.a[9];
    const int r = t / q_len;
    contiguous_base = (size_t)r * kv_len;
    lim = kv_len - q_len + (t - r * q_len) + 1;
  }
  const int k_begin = split * kMlaSplit, k_end = min(k_begin + kMlaSplit, lim);
  __nv_bfloat16 *po = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  float *plse = reinterpret_cast<float *>(d.p[3]);
  if (k_begin >= k_end) {   // nothing to see in this split: the merge skips it
    if (tid < 16) plse[((size_t)t * H + head0 + tid) * S + split] = -INFINITY;
    return;
  }
  uint8_t *Qs = c.s.xtile;
  uint8_t *KVs = Qs + 16 * kMlaRow;
  uint8_t *Ps = KVs + kMlaSub * kMlaRow;
  float *mx = reinterpret_cast<float *>(Ps + 16 * kMlaPRow);   // [8 warps][16 rows]
  float *sm = mx + 8 * 16;
  const __nv_bfloat16 *cache = reinterpret_cast<const __nv_bfloat16 *>(d.p[1]);
  {
    const __nv_bfloat16 *qg = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]) + (size_t)t * ldq + (size_t)head0 * kMlaDk;
    for (int i = tid; i < 16 * (kMlaDk / 8); i += kConsumerThreads) {
      const int h = i / (kMlaDk / 8), v = i - h * (kMlaDk / 8);
      *reinterpret_cast<uint4 *>(Qs + (size_t)h * kMlaRow + (size_t)v * 16) =
          __ldcg(reinterpret_cast<const uint4 *>(qg + (size_t)h * kMlaDk) + v);
    }
  }
  float o[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // running max / sum of rows g and g + 8
  const uint32_t q_addr = smem_u32(Qs) + (uint32_t)(lane & 15) * kMlaRow + (uint32_t)(lane >> 4) * 16u;
  const uint32_t k_addr = smem_u32(KVs) + (uint32_t)(warp * 8 + g) * kMlaRow + (uint32_t)q * 4u;
  const uint32_t p_addr = smem_u32(Ps) + (uint32_t)(lane & 15) * kMlaPRow + (uint32_t)(lane >> 4) * 16u;
  const uint32_t v_addr = smem_u32(KVs) + (uint32_t)(((lane >> 3) & 1) * 8 + (lane & 7)) * kMlaRow +
                          (uint32_t)(warp * 64 + (lane >> 4) * 8) * 2u;
  for (int sub = k_begin; sub < k_end; sub += kMlaSub) {
    const int nrows = min(kMlaSub, k_end - sub);
    consumer_sync();   // the previous tile (and the q tile of the previous task) is no longer read
    {
      // four threads per kv row: one page-table lookup, then 18 asynchronous 16-byte copies straight into
      // shared memory (no registers held, all in flight together); rows past the end are zero-filled
      const int r = tid >> 2, part = tid & 3;
      const uint32_t dst = smem_u32(KVs + (size_t)r * kMlaRow) + (uint32_t)part * 288u;
      if (r < nrows) {
        const int pos = sub + r;
        size_t row;
        if (page > 0) {
          const int pid = __ldcg(&P.meta.paged_kv_indices[kv0 + pos / page]);
          row = (size_t)pid * page + pos % page;
        } else {
          row = contiguous_base + pos;
        }
        const uint8_t *src = reinterpret_cast<const uint8_t *>(cache + row * kMlaDk) + part * 288;
#pragma unroll
        for (int j = 0; j < 18; ++j)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + j * 16u), "l"(src + j * 16) : "memory");
      } else {
#pragma unroll
        for (int j = 0; j < 18; ++j)
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst + j * 16u), "r"(0u) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    consumer_sync();
    // scores of this warp's 8 kv rows
    float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int ks = 0; ks < kMlaDk / 16; ++ks) {
      uint32_t a[4], b0, b1;
      ldmatrix_x4(a, q_addr + (uint32_t)ks * 32u);
      asm volatile("ld.shared.b32 %0, [%1];" : "=r"(b0) : "r"(k_addr + (uint32_t)ks * 32u));
      asm volatile("ld.shared.b32 %0, [%1];" : "=r"(b1) : "r"(k_addr + (uint32_t)ks * 32u + 16u));
      mma_bf16_16816(sacc, a, b0, b1);
    }
    const int j0 = warp * 8 + 2 * q;
    const bool v0 = j0 < nrows, v1 = j0 + 1 < nrows;
    sacc[0] = v0 ? sacc[0] * scale : -INFINITY;
    sacc[1] = v1 ? sacc[1] * scale : -INFINITY;
    sacc[2] = v0 ? sacc[2] * scale : -INFINITY;
    sacc[3] = v1 ? sacc[3] * scale : -INFINITY;
    float r0 = fmaxf(sacc[0], sacc[1]), r1 = fmaxf(sacc[2], sacc[3]);
    r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, 1));
    r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, 2));
    r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, 1));
    r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, 2));
    if (q == 0) { mx[warp * 16 + g] = r0; mx[warp * 16 + g + 8] = r1; }
    consumer_sync();
    float n0 = m0, n1 = m1;
#pragma unroll
    for (int w = 0; w < 8; ++w) { n0 = fmaxf(n0, mx[w * 16 + g]); n1 = fmaxf(n1, mx[w * 16 + g + 8]); }
    const float p00 = __expf(sacc[0] - n0), p01 = __expf(sacc[1] - n0);   // exp(-inf) = 0 for masked rows
    const float p10 = __expf(sacc[2] - n1), p11 = __expf(sacc[3] - n1);
    float s0 = p00 + p01, s1 = p10 + p11;
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    if (q == 0) { sm[warp * 16 + g] = s0; sm[warp * 16 + g + 8] = s1; }
    {
      const __nv_bfloat162 w0 = __floats2bfloat162_rn(p00, p01), w1 = __floats2bfloat162_rn(p10, p11);
      *reinterpret_cast<__nv_bfloat162 *>(Ps + (size_t)g * kMlaPRow + (size_t)j0 * 2) = w0;
      *reinterpret_cast<__nv_bfloat162 *>(Ps + (size_t)(g + 8) * kMlaPRow + (size_t)j0 * 2) = w1;
    }
    consumer_sync();
    const float al0 = __expf(m0 - n0), al1 = __expf(m1 - n1);   // 0 on the first tile (m = -inf)
    float t0 = 0.f, t1 = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { t0 += sm[w * 16 + g]; t1 += sm[w * 16 + g + 8]; }
    l0 = l0 * al0 + t0;
    l1 = l1 * al1 + t1;
    m0 = n0;
    m1 = n1;
#pragma unroll
    for (int i = 0; i < 8; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
    // O[:, 64 warp ...] += P . V
#pragma unroll
    for (int ks = 0; ks < kMlaSub / 16; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a, p_addr + (uint32_t)ks * 32u);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, v_addr + (uint32_t)(ks * 16) * kMlaRow + (uint32_t)np * 32u);
        mma_bf16_16816(o[2 * np], a, b[0], b[1]);
        mma_bf16_16816(o[2 * np + 1], a, b[2], b[3]);
      }
    }
  }
  const float i0 = __fdividef(1.0f, l0), i1 = __fdividef(1.0f, l1);
  const size_t row0 = ((size_t)t * H + head0 + g) * S + split, row1 = ((size_t)t * H + head0 + g + 8) * S + split;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int col = warp * 64 + i * 8 + 2 * q;
    *reinterpret_cast<__nv_bfloat162 *>(po + row0 * kMlaDv + col) = __floats2bfloat162_rn(o[i][0] * i0, o[i][1] * i0);
    *reinterpret_cast<__nv_bfloat162 *>(po + row1 * kMlaDv + col) = __floats2bfloat162_rn(o[i][2] * i1, o[i][3] * i1);
  }
  if (warp == 0 && q == 0) {
    plse[row0] = m0 + __logf(l0);
    plse[row1] = m1 + __logf(l1);
  }
}

// TASK_MLA_REDUCE: out[token, head] = sum_s w_s O_s with w_s = exp(lse_s - max) / sum: one warp per (token, head) row
// (mla_reduce_sm100.cuh:28-76 / mla_mtp_reduce).
__device__ void run_mla_reduce(const Ctx &c, const TaskDesc &d) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = d.a[2], S = d.a[3], ldo = d.a[4];
  const int r1 = min(d.a[1], active_tokens(c.P) * H);
  const __nv_bfloat16 *po = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  const float *plse = reinterpret_cast<const float *>(d.p[1]);
  __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  for (int row = d.a[0] + warp; row < r1; row += kConsumerThreads / 32) {
    // lane s keeps the weights of splits s and s + 32 (S <= 64); the O rows of four splits are fetched together
    const float ls0 = lane < S ? __ldcg(&plse[(size_t)row * S + lane]) : -INFINITY;
    const float ls1 = lane + 32 < S ? __ldcg(&plse[(size_t)row * S + lane + 32]) : -INFINITY;
    float mxv = fmaxf(ls0, ls1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mxv = fmaxf(mxv, __shfl_xor_sync(0xffffffffu, mxv, o));
    const float w0 = ls0 == -INFINITY ? 0.f : __expf(ls0 - mxv), w1 = ls1 == -INFINITY ? 0.f : __expf(ls1 - mxv);
    float tot = w0 + w1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (int s0 = 0; s0 < S; s0 += 4) {
      float w[4];
      uint4 x0[4], x1[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int s = s0 + u;
        w[u] = __shfl_sync(0xffffffffu, s < 32 ? w0 : w1, s & 31);
        if (s >= S) w[u] = 0.f;
        x0[u] = x1[u] = make_uint4(0, 0, 0, 0);
        if (w[u] != 0.f) {
          const uint4 *src = reinterpret_cast<const uint4 *>(po + ((size_t)row * S + s) * kMlaDv + lane * 16);
          x0[u] = __ldcg(src);
          x1[u] = __ldcg(src + 1);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t xs[8] = {x0[u].x, x0[u].y, x0[u].z, x0[u].w, x1[u].x, x1[u].y, x1[u].z, x1[u].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          acc[2 * i] += w[u] * __uint_as_float(xs[i] << 16);
          acc[2 * i + 1] += w[u] * __uint_as_float(xs[i] & 0xffff0000u);
        }
      }
    }
    const float inv = tot > 0.f ? __fdividef(1.0f, tot) : 0.f;
    const int tok = row / H, h = row - tok * H;
    __nv_bfloat16 *dst = out + (size_t)tok * ldo + (size_t)h * kMlaDv + lane * 16;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      *reinterpret_cast<__nv_bfloat162 *>(dst + 2 * i) = __floats2bfloat162_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
  }
}

// ---------------------------------------------------------------------------
// TASK_ATTENTION: paged split-KV GQA decode attention with fused QK-norm, RoPE, KV append
// ---------------------------------------------------------------------------
// One task = (request slot, kv head, kv chunk).  Work that does not depend on this layer's qkv
// projection -- the request's page table and the K/V rows already in the cache -- is fetched into
// registers BEFORE the task waits for its dependency, so that after the wait only the new token's
// q/k/v have to be loaded.  Partial results of the chunks are merged by the last chunk to finish.
struct ReqView {
  int q0, nq, kv0, seq_len;
};

constexpr int kAttnPre = 4;   // kv rows per half-warp fetched ahead of the dependency (64 rows per CTA)

struct AttnPre {
  ReqView rv;
  int start, end, new_start, n_active;
  uint4 k[kAttnPre], v[kAttnPre];
  uint2 cs0, sn0;   // rotary cos / sin of the first new position (this lane's dims)
};

__device__ __forceinline__ ReqView request_view(const KernelParams &P, const TaskDesc &d) {
  ReqView r;
  const int slot = d.a[A_SLOT];
  if (d.a[A_FLAGS] & 4) {   // contiguous cache: one token per slot, length = step + 1
    r.q0 = slot;
    r.nq = (slot < active_tokens(P)) ? 1 : 0;
    r.kv0 = 0;
    r.seq_len = P.meta.step ? __ldcg(&P.meta.step[slot]) + 1 : 1;
    return r;
  }
  r.q0 = __ldcg(&P.meta.qo_indptr[slot]);
  r.nq = __ldcg(&P.meta.qo_indptr[slot + 1]) - r.q0;
  r.kv0 = __ldcg(&P.meta.paged_kv_indptr[slot]);
  const int npages = __ldcg(&P.meta.paged_kv_indptr[slot + 1]) - r.kv0;
  r.seq_len = (npages - 1) * d.a[A_PAGE] + __ldcg(&P.meta.paged_kv_last_page_len[slot]);
  return r;
}

// element offset of (position, kv head) inside a [pages, page, Hkv, 128] cache
__device__ __forceinline__ size_t kv_offset(const KernelParams &P, const TaskDesc &d, const ReqView &rv, int pos) {
  const int page = d.a[A_PAGE];
  const int hkv = d.a[A_HKV];
  if (d.a[A_FLAGS] & 4)
    return (((size_t)d.a[A_SLOT] * d.a[A_CSEQ] + pos) * hkv + d.a[A_HEAD]) * 128;
  const int pidx = pos / page;
  const int pid = __ldcg(&P.meta.paged_kv_indices[rv.kv0 + pidx]);
  return (((size_t)pid * page + (pos - pidx * page)) * hkv + d.a[A_HEAD]) * 128;
}

// Issued by the streaming warp when it walks past an attention task, i.e. while the compute warps are
// still a few chunks away from it: pulls the cached K/V rows of the task's chunk into L2.  The batch
// description may still be the previous iteration's when this runs early in a launch; every index read
// here stays inside its buffer for any mix of old and new values, and a stale prefetch is harmless.
//
// It also leaves the request's description and the page ids of the chunk's first 64 positions in shared memory
// (`attention stash`, the unused tail of the full-barrier array) for the compute warps, which would otherwise pay
// two dependent L2 round trips for them right before their dependency wait.  The stash is published only when the
// batching event of this iteration had already fired (acquire), i.e. when what was read is final; it carries the task
// index, is written index-last and read index-first-and-last, so a reader either gets a consistent record of its own
// task or falls back to its own loads.
// Where the stash record of a task lives: the narrow instantiation has one record in the unused tail of the
// full-barrier array; the general one, whose workers see runs of many attention tasks that the streaming warp walks
// past at once, has a ring of kStashRing records after the flags.
template <bool GENERAL>
__device__ __forceinline__ volatile int *attention_stash(const Ctx &c, int task) {
  if (GENERAL) return reinterpret_cast<volatile int *>(c.s.flags + 16) + (task & (kStashRing - 1)) * 8;
  return reinterpret_cast<volatile int *>(&c.s.full[8]);
}

template <bool GENERAL>
__device__ void prefetch_attention_kv_l2(const Ctx &c, const TaskDesc *d, int lane, int task) {
  const KernelParams &P = c.P;
  if ((d->a[A_FLAGS] & 4) || P.meta.qo_indptr == nullptr) return;
  const bool final_meta = P.meta_static || ld_acquire_gpu(&P.counters[0]) >= c.iteration;
  const int slot = d->a[A_SLOT];
  const int q0 = __ldcg(&P.meta.qo_indptr[slot]);
  const int nq = __ldcg(&P.meta.qo_indptr[slot + 1]) - q0;
  const int kv0 = __ldcg(&P.meta.paged_kv_indptr[slot]);
  const int npages = __ldcg(&P.meta.paged_kv_indptr[slot + 1]) - kv0;
  const int page = d->a[A_PAGE], hkv = d->a[A_HKV];
  if (nq <= 0 || npages <= 0 || kv0 < 0 || kv0 + npages > P.max_num_pages) return;
  const int seq_len = (npages - 1) * page + min(max(__ldcg(&P.meta.paged_kv_last_page_len[slot]), 1), page);
  const int NC = d->a[A_NCHUNK];
  int L = (seq_len + NC - 1) / NC;
  L = (L + 15) & ~15;
  const int start = d->a[A_CHUNK] * L;
  const int old_end = min(min(seq_len, start + L), seq_len - nq);
  const char *kc = reinterpret_cast<const char *>(d->p[1]);
  const char *vc = reinterpret_cast<const char *>(d->p[2]);
  if (final_meta && page >= 64 && start < seq_len) {
    const int pb = start / page;
    const int p0 = __ldcg(&P.meta.paged_kv_indices[kv0 + pb]);
    const int p1 = (pb + 1 < npages) ? __ldcg(&P.meta.paged_kv_indices[kv0 + pb + 1]) : p0;
    if (lane == 0) {
      volatile int *st = attention_stash<GENERAL>(c, task);
      st[0] = -1;
      __threadfence_block();
      st[1] = q0; st[2] = nq; st[3] = kv0; st[4] = (npages - 1) * page + __ldcg(&P.meta.paged_kv_last_page_len[slot]);
      st[5] = pb; st[6] = p0; st[7] = p1;
      __threadfence_block();
      st[0] = task;
    }
  }
  // The general instantiation streams the chunk through shared memory with many copies in flight: an L2 prefetch
  // ahead of it only fetches every row twice whenever the rows do not survive in L2 until they are used (measured:
  // DRAM reads 1.87 x the K/V bytes on a 268 MB attention-only launch).
  for (int pos = start + lane; !GENERAL && pos < old_end; pos += 32) {
    const int pidx = pos / page;
    const int pid = min(max(__ldcg(&P.meta.paged_kv_indices[kv0 + pidx]), 0), P.max_num_pages - 1);
    const size_t off = ((((size_t)pid * page + (pos - pidx * page)) * hkv + d->a[A_HEAD]) * 128) * 2;
    asm volatile("prefetch.global.L2 [%0];" ::"l"(kc + off));
    asm volatile("prefetch.global.L2 [%0];" ::"l"(kc + off + 128));
    asm volatile("prefetch.global.L2 [%0];" ::"l"(vc + off));
    asm volatile("prefetch.global.L2 [%0];" ::"l"(vc + off + 128));
  }
}

__device__ __forceinline__ void load_rope(const __nv_bfloat16 *cosT, const __nv_bfloat16 *sinT, int pos, int rows,
                                          int lane, uint2 &cs, uint2 &sn);

// Runs before the dependency wait (the batch description is already final).
template <bool GENERAL>
__device__ __forceinline__ void attention_prefetch(const Ctx &c, const TaskDesc &d, AttnPre &pre, int task) {
  const KernelParams &P = c.P;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // the streaming warp may have left this task's request description and first page ids in shared memory
  const volatile int *st = attention_stash<GENERAL>(c, task);
  bool hit = st[0] == task;
  int pb = 0, p0 = 0, p1 = 0;
  if (hit) {
    pre.rv.q0 = st[1]; pre.rv.nq = st[2]; pre.rv.kv0 = st[3]; pre.rv.seq_len = st[4];
    pb = st[5]; p0 = st[6]; p1 = st[7];
    __threadfence_block();
    hit = st[0] == task;
  }
  if (!hit) pre.rv = request_view(P, d);
  const int NC = d.a[A_NCHUNK];
  int L = (pre.rv.seq_len + NC - 1) / NC;
  L = (L + 15) & ~15;
  pre.n_active = pre.rv.nq > 0 ? (pre.rv.seq_len + L - 1) / L : 0;
  pre.start = d.a[A_CHUNK] * L;
  pre.end = min(pre.rv.seq_len, pre.start + L);
  pre.new_start = pre.rv.seq_len - pre.rv.nq;
  pre.cs0 = pre.sn0 = make_uint2(0, 0);
  if (pre.rv.nq <= 0) return;
  load_rope((d.a[A_FLAGS] & 2) ? reinterpret_cast<const __nv_bfloat16 *>(d.p[5]) : nullptr,
            reinterpret_cast<const __nv_bfloat16 *>(d.p[6]), pre.new_start, d.a[A_ROPE_ROWS], lane, pre.cs0, pre.sn0);
  const __nv_bfloat16 *kc = reinterpret_cast<const __nv_bfloat16 *>(d.p[1]);
  const __nv_bfloat16 *vc = reinterpret_cast<const __nv_bfloat16 *>(d.p[2]);
  const int hw = lane >> 4, hl = lane & 15;
  const int old_end = min(pre.end, pre.new_start);
#pragma unroll
  for (int i = 0; i < kAttnPre; ++i) {
    const int pos = pre.start + warp * 2 + hw + 16 * i;
    // Rows outside the range get defined zeros: every row is read later (masked), and leaving them
    // indeterminate would let the compiler make these loads unconditional, i.e. read out of range.
    pre.k[i] = make_uint4(0, 0, 0, 0);
    pre.v[i] = make_uint4(0, 0, 0, 0);
    if (pos < old_end) {
      size_t off;
      if (hit) {   // positions start .. start + 63 lie in the page of `start` or the next one (pages hold >= 64 rows)
        const int page = d.a[A_PAGE], pidx = pos / page;
        off = (((size_t)(pidx == pb ? p0 : p1) * page + (pos - pidx * page)) * d.a[A_HKV] + d.a[A_HEAD]) * 128 + hl * 8;
      } else {
        off = kv_offset(P, d, pre.rv, pos) + hl * 8;
      }
      pre.k[i] = __ldcs(reinterpret_cast<const uint4 *>(kc + off));
      pre.v[i] = __ldcs(reinterpret_cast<const uint4 *>(vc + off));
    }
  }
}

// One warp: RMS-normalise (optional) and rotate (optional) a 128-wide head vector.
// Lane l holds elements 4l..4l+3.  Norm result is rounded to bf16 before the rotation,
// as include/mirage/persistent_kernel/tasks/blackwell/norm_sm100.cuh:96-126 does.
__device__ __forceinline__ void norm_rope_head(float (&x)[4], const __nv_bfloat16 *norm_w, float eps, bool rope,
                                               uint2 cs, uint2 sn, int lane) {
  if (norm_w) {
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss * (1.0f / 128.0f) + eps);
    const uint2 nw = __ldg(reinterpret_cast<const uint2 *>(norm_w + lane * 4));
    const float w[4] = {bf16_lo(nw.x), bf16_hi(nw.x), bf16_lo(nw.y), bf16_hi(nw.y)};
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = round_bf16(x[i] * inv * w[i]);
  }
  if (rope) {
    const float cf[4] = {bf16_lo(cs.x), bf16_hi(cs.x), bf16_lo(cs.y), bf16_hi(cs.y)};
    const float sf[4] = {bf16_lo(sn.x), bf16_hi(sn.x), bf16_lo(sn.y), bf16_hi(sn.y)};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);   // element d +/- 64
      const float rot = (lane < 16) ? -other : other;
      x[i] = round_bf16(x[i] * cf[i] + rot * sf[i]);
    }
  }
}

// cos / sin of one position for this lane's four dims (zeros when the layer has no rotary embedding)
__device__ __forceinline__ void load_rope(const __nv_bfloat16 *cosT, const __nv_bfloat16 *sinT, int pos, int rows,
                                          int lane, uint2 &cs, uint2 &sn) {
  cs = sn = make_uint2(0, 0);
  if (cosT) {
    const size_t o = (size_t)min(pos, rows - 1) * 128 + lane * 4;
    cs = __ldg(reinterpret_cast<const uint2 *>(cosT + o));
    sn = __ldg(reinterpret_cast<const uint2 *>(sinT + o));
  }
}

template <int G>
struct AttnState {
  float m[G], l[G], o[G][8];
};

// one kv row (8 of its 128 dims per lane) against the G query heads of this kv head
template <int G>
__device__ __forceinline__ void attn_row(AttnState<G> &s, const float (&q)[G][8], const uint4 &kr, const uint4 &vr,
                                         unsigned hmask) {
  const float kf[8] = {bf16_lo(kr.x), bf16_hi(kr.x), bf16_lo(kr.y), bf16_hi(kr.y),
                       bf16_lo(kr.z), bf16_hi(kr.z), bf16_lo(kr.w), bf16_hi(kr.w)};
  const float vf[8] = {bf16_lo(vr.x), bf16_hi(vr.x), bf16_lo(vr.y), bf16_hi(vr.y),
                       bf16_lo(vr.z), bf16_hi(vr.z), bf16_lo(vr.w), bf16_hi(vr.w)};
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float sc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sc = fmaf(q[g][i], kf[i], sc);
    sc += __shfl_xor_sync(hmask, sc, 8);
    sc += __shfl_xor_sync(hmask, sc, 4);
    sc += __shfl_xor_sync(hmask, sc, 2);
    sc += __shfl_xor_sync(hmask, sc, 1);
    const float mn = fmaxf(s.m[g], sc);
    const float corr = exp2f(s.m[g] - mn);
    const float p = exp2f(sc - mn);
    s.m[g] = mn;
    s.l[g] = s.l[g] * corr + p;
#pragma unroll
    for (int i = 0; i < 8; ++i) s.o[g][i] = fmaf(p, vf[i], s.o[g][i] * corr);
  }
}

// Up to four kv rows at once: the dot products and their shuffle reductions are independent chains, and the
// running softmax state is updated once for the whole batch.
template <int G>
__device__ __forceinline__ void attn_rows4(AttnState<G> &s, const float (&q)[G][8], const uint4 (&kr)[kAttnPre],
                                           const uint4 (&vr)[kAttnPre], int nrows, unsigned hmask) {
  float sc[kAttnPre][G];
#pragma unroll
  for (int i = 0; i < kAttnPre; ++i) {
    const float kf[8] = {bf16_lo(kr[i].x), bf16_hi(kr[i].x), bf16_lo(kr[i].y), bf16_hi(kr[i].y),
                         bf16_lo(kr[i].z), bf16_hi(kr[i].z), bf16_lo(kr[i].w), bf16_hi(kr[i].w)};
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float a = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) a = fmaf(q[g][e], kf[e], a);
      sc[i][g] = a;
    }
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1)
#pragma unroll
    for (int i = 0; i < kAttnPre; ++i)
#pragma unroll
      for (int g = 0; g < G; ++g) sc[i][g] += __shfl_xor_sync(hmask, sc[i][g], o);
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float mn = s.m[g];
#pragma unroll
    for (int i = 0; i < kAttnPre; ++i)
      if (i < nrows) mn = fmaxf(mn, sc[i][g]);
    const float corr = exp2f(s.m[g] - mn);
    float p[kAttnPre];
    float psum = 0.f;
#pragma unroll
    for (int i = 0; i < kAttnPre; ++i) {
      p[i] = (i < nrows) ? exp2f(sc[i][g] - mn) : 0.f;
      psum += p[i];
    }
    s.m[g] = mn;
    s.l[g] = s.l[g] * corr + psum;
#pragma unroll
    for (int e = 0; e < 8; ++e) s.o[g][e] *= corr;
#pragma unroll
    for (int i = 0; i < kAttnPre; ++i) {
      const float vf[8] = {bf16_lo(vr[i].x), bf16_hi(vr[i].x), bf16_lo(vr[i].y), bf16_hi(vr[i].y),
                           bf16_lo(vr[i].z), bf16_hi(vr[i].z), bf16_lo(vr[i].w), bf16_hi(vr[i].w)};
#pragma unroll
      for (int e = 0; e < 8; ++e) s.o[g][e] = fmaf(p[i], vf[e], s.o[g][e]);
    }
  }
}

template <int GT>
__device__ __forceinline__ void attention_body(const Ctx &c, const TaskDesc &d, const AttnPre &pre, const int G,
                                               int task) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const ReqView rv = pre.rv;
  if (rv.nq <= 0) return;
  const int NC = d.a[A_NCHUNK], chunk = d.a[A_CHUNK], head = d.a[A_HEAD];
  const int hq = d.a[A_HQ];
  const int flags = d.a[A_FLAGS];
  const float eps = __int_as_float(d.a[A_EPS]);
  const __nv_bfloat16 *qkv = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  __nv_bfloat16 *kc = reinterpret_cast<__nv_bfloat16 *>(d.p[1]);
  __nv_bfloat16 *vc = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  const __nv_bfloat16 *qn = (flags & 1) ? reinterpret_cast<const __nv_bfloat16 *>(d.p[3]) : nullptr;
  const __nv_bfloat16 *kn = (flags & 1) ? reinterpret_cast<const __nv_bfloat16 *>(d.p[4]) : nullptr;
  const __nv_bfloat16 *cosT = (flags & 2) ? reinterpret_cast<const __nv_bfloat16 *>(d.p[5]) : nullptr;
  const __nv_bfloat16 *sinT = (flags & 2) ? reinterpret_cast<const __nv_bfloat16 *>(d.p[6]) : nullptr;
  __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[7]);
  const int ldq = d.a[A_LDQKV], ldo = d.a[A_LDO];
  const int rope_rows = d.a[A_ROPE_ROWS];
  const int start = pre.start, end = pre.end, new_start = pre.new_start, n_active = pre.n_active;
  const size_t head_base = (size_t)head * (G + 2) * 128;

  const bool aprof = P.profiler != nullptr && (uint64_t)(task + 1) * 8 <= P.profiler_entries;
  float *q_s = reinterpret_cast<float *>(c.s.xtile);            // [G][128], pre-scaled
  float *w_ml = q_s + G * 128;                                    // [8 warps][G][2]
  float *w_o = w_ml + 8 * G * 2;                                  // [8 warps][G][128]
  uint2 *new_kv = reinterpret_cast<uint2 *>(w_o + 8 * G * 128);   // [nq][k 32 lanes | v 32 lanes] (4 bf16 per lane)

  // ---- append the new keys / values that fall into this chunk (cache + shared-memory copy) ----
  for (int pos = max(start, new_start) + warp; pos < end; pos += 8) {
    const int tok = rv.q0 + (pos - new_start);
    const __nv_bfloat16 *kp = qkv + (size_t)tok * ldq + head_base + (size_t)G * 128 + lane * 4;
    const uint2 kr = __ldcg(reinterpret_cast<const uint2 *>(kp));
    const uint2 vr = __ldcg(reinterpret_cast<const uint2 *>(kp + 128));
    float x[4] = {bf16_lo(kr.x), bf16_hi(kr.x), bf16_lo(kr.y), bf16_hi(kr.y)};
    uint2 cs = pre.cs0, sn = pre.sn0;
    if (pos != new_start) load_rope(cosT, sinT, pos, rope_rows, lane, cs, sn);
    norm_rope_head(x, kn, eps, cosT != nullptr, cs, sn, lane);
    const uint2 kw = make_uint2(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]));
    const size_t off = kv_offset(P, d, rv, pos) + lane * 4;
    *reinterpret_cast<uint2 *>(kc + off) = kw;
    *reinterpret_cast<uint2 *>(vc + off) = vr;
    new_kv[(size_t)(pos - new_start) * 64 + lane] = kw;
    new_kv[(size_t)(pos - new_start) * 64 + 32 + lane] = vr;
  }

  const float qscale = 0.08838834764831845f * 1.4426950408889634f;   // 1/sqrt(128) * log2(e)
  const int hw = lane >> 4;          // half-warp
  const int hl = lane & 15;          // lane within the half-warp: dims hl*8 .. hl*8+7
  const unsigned hmask = hw ? 0xffff0000u : 0x0000ffffu;
  const int old_end = min(end, new_start);

  for (int t = 0; t < rv.nq; ++t) {
    const int pq = new_start + t;
    const int tok = rv.q0 + t;
    const int lim = min(end, pq + 1);
    if (warp < G) {
      const __nv_bfloat16 *qp = qkv + (size_t)tok * ldq + head_base + (size_t)warp * 128 + lane * 4;
      const uint2 qr = __ldcg(reinterpret_cast<const uint2 *>(qp));
      float x[4] = {bf16_lo(qr.x), bf16_hi(qr.x), bf16_lo(qr.y), bf16_hi(qr.y)};
      uint2 cs = pre.cs0, sn = pre.sn0;
      if (t != 0) load_rope(cosT, sinT, pq, rope_rows, lane, cs, sn);
      norm_rope_head(x, qn, eps, cosT != nullptr, cs, sn, lane);
      *reinterpret_cast<float4 *>(&q_s[warp * 128 + lane * 4]) =
          make_float4(x[0] * qscale, x[1] * qscale, x[2] * qscale, x[3] * qscale);
    }
    consumer_sync();   // q_s and new_kv are ready
    if (tid == 0 && aprof && t == 0) P.profiler[(size_t)task * 8 + 4] = globaltimer_ns();
    const int first = start + warp * 2 + hw;
    for (int gb = 0; gb < G; gb += GT) {   // GT query heads at a time keeps the register footprint bounded
      float q[GT][8];
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        const float4 a = *reinterpret_cast<const float4 *>(&q_s[(gb + g) * 128 + hl * 8]);
        const float4 b = *reinterpret_cast<const float4 *>(&q_s[(gb + g) * 128 + hl * 8 + 4]);
        q[g][0] = a.x; q[g][1] = a.y; q[g][2] = a.z; q[g][3] = a.w;
        q[g][4] = b.x; q[g][5] = b.y; q[g][6] = b.z; q[g][7] = b.w;
      }
      AttnState<GT> s;
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        s.m[g] = -INFINITY;
        s.l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s.o[g][i] = 0.f;
      }
      // rows fetched ahead of the dependency (positions first, first + 16, ...: a prefix of them is valid)
      {
        const int bound = min(old_end, lim);
        const int nrows = first < bound ? min((bound - first + 15) >> 4, kAttnPre) : 0;
        if (nrows > 0) attn_rows4<GT>(s, q, pre.k, pre.v, nrows, hmask);   // uniform per half-warp
      }
      if (tid == 0 && aprof && t == 0 && gb == 0) P.profiler[(size_t)task * 8 + 5] = globaltimer_ns();
      // remaining old rows of a long chunk
      for (int pos = first + 16 * kAttnPre; pos < min(old_end, lim); pos += 16) {
        const size_t off = kv_offset(P, d, rv, pos) + hl * 8;
        const uint4 kr = __ldcs(reinterpret_cast<const uint4 *>(kc + off));
        const uint4 vr = __ldcs(reinterpret_cast<const uint4 *>(vc + off));
        attn_row<GT>(s, q, kr, vr, hmask);
      }
      // rows appended by this task: read back from shared memory
      {
        int pos = first;
        if (pos < new_start) pos += ((new_start - pos + 15) / 16) * 16;
        for (; pos < lim; pos += 16) {
          const uint4 kr = *reinterpret_cast<const uint4 *>(&new_kv[(size_t)(pos - new_start) * 64 + hl * 2]);
          const uint4 vr = *reinterpret_cast<const uint4 *>(&new_kv[(size_t)(pos - new_start) * 64 + 32 + hl * 2]);
          attn_row<GT>(s, q, kr, vr, hmask);
        }
      }
      if (tid == 0 && aprof && t == 0 && gb == 0) P.profiler[(size_t)task * 8 + 6] = globaltimer_ns();
      __syncwarp();
      // fold the two half-warps together
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        const float m2 = __shfl_xor_sync(0xffffffffu, s.m[g], 16);
        const float l2 = __shfl_xor_sync(0xffffffffu, s.l[g], 16);
        const float mn = fmaxf(s.m[g], m2);
        const float c1 = (s.m[g] == -INFINITY) ? 0.f : exp2f(s.m[g] - mn);
        const float c2 = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mn);
        s.l[g] = s.l[g] * c1 + l2 * c2;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float o2 = __shfl_xor_sync(0xffffffffu, s.o[g][i], 16);
          s.o[g][i] = s.o[g][i] * c1 + o2 * c2;
        }
        s.m[g] = mn;
        if (hw == 0) {
          float4 *wo = reinterpret_cast<float4 *>(&w_o[((size_t)warp * G + gb + g) * 128 + hl * 8]);
          wo[0] = make_float4(s.o[g][0], s.o[g][1], s.o[g][2], s.o[g][3]);
          wo[1] = make_float4(s.o[g][4], s.o[g][5], s.o[g][6], s.o[g][7]);
          if (hl == 0) {
            w_ml[(warp * G + gb + g) * 2 + 0] = s.m[g];
            w_ml[(warp * G + gb + g) * 2 + 1] = s.l[g];
          }
        }
      }
    }
    if (tid == 0 && aprof && t == 0) P.profiler[(size_t)task * 8 + 7] = globaltimer_ns();
    consumer_sync();
    // combine the 8 warps; thread -> (g, dim) pairs
    for (int idx = tid; idx < G * 128; idx += kConsumerThreads) {
      const int g = idx >> 7, dd = idx & 127;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 8; ++w) M = fmaxf(M, w_ml[(w * G + g) * 2]);
      float Ls = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float mw = w_ml[(w * G + g) * 2];
        const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        Ls += w_ml[(w * G + g) * 2 + 1] * sc;
        O += w_o[((size_t)w * G + g) * 128 + dd] * sc;
      }
      const int hq_idx = head * G + g;
      if (NC == 1) {
        out[(size_t)tok * ldo + (size_t)hq_idx * 128 + dd] = __float2bfloat16_rn(Ls > 0.f ? O / Ls : 0.f);
      } else {
        const size_t base = ((size_t)tok * hq + hq_idx) * NC + chunk;
        __stcg(&P.attn_scratch[base * 130 + 2 + dd], O);
        if (dd == 0) {
          __stcg(&P.attn_scratch[base * 130 + 0], M);
          __stcg(&P.attn_scratch[base * 130 + 1], Ls);
        }
      }
    }
    if (t + 1 < rv.nq) consumer_sync();   // q_s / w_o are rewritten for the next query token
  }
  if (NC == 1) return;
  // ---- split-KV merge by the last chunk task to arrive ---------------------------
  consumer_sync();
  if (tid == 0) {
    unsigned int old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;"
                 : "=r"(old)
                 : "l"(&P.attn_tickets[d.a[A_TICKET] + d.a[A_SLOT] * d.a[A_HKV] + head])
                 : "memory");
    c.s.flags[1] = ((old + 1u) % (unsigned)NC == 0u) ? 1 : 0;
  }
  consumer_sync();
  if (c.s.flags[1] == 0) return;
  // Merge: one warp per 32 consecutive output dims of a (token, head).  Lane c fetches chunk c's (max, sum)
  // while every lane fetches its dim of all chunks; all loads are in flight together (a single round trip to
  // L2), then the weights are formed with shuffles.  NC <= 32.
  for (int item = warp; item < rv.nq * G * 4; item += 8) {
    const int row = item >> 2, dd = ((item & 3) << 5) + lane;
    const int t = row / G, g = row - t * G;
    const int tok = rv.q0 + t;
    const int hq_idx = head * G + g;
    const size_t base = ((size_t)tok * hq + hq_idx) * NC;
    const bool v = lane < n_active;
    const float m = v ? __ldcg(&P.attn_scratch[(base + lane) * 130]) : -INFINITY;
    const float l = v ? __ldcg(&P.attn_scratch[(base + lane) * 130 + 1]) : 0.f;
    float ow[16], ow2[16];
#pragma unroll
    for (int u = 0; u < 16; ++u)
      ow[u] = (u < n_active) ? __ldcg(&P.attn_scratch[(base + u) * 130 + 2 + dd]) : 0.f;
    if (n_active > 16) {
#pragma unroll
      for (int u = 0; u < 16; ++u)
        ow2[u] = (16 + u < n_active) ? __ldcg(&P.attn_scratch[(base + 16 + u) * 130 + 2 + dd]) : 0.f;
    }
    float M = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
    const float Ls = warp_sum(l * w);
    float O = 0.f;
#pragma unroll
    for (int u = 0; u < 16; ++u) O = fmaf(ow[u], __shfl_sync(0xffffffffu, w, u), O);
    if (n_active > 16) {
#pragma unroll
      for (int u = 0; u < 16; ++u) O = fmaf(ow2[u], __shfl_sync(0xffffffffu, w, 16 + u), O);
    }
    out[(size_t)tok * ldo + (size_t)hq_idx * 128 + dd] = __float2bfloat16_rn(Ls > 0.f ? O / Ls : 0.f);
  }
}

__device__ __forceinline__ void run_attention(const Ctx &c, const TaskDesc &d, const AttnPre &pre, int task) {
  const int G = d.a[A_HQ] / d.a[A_HKV];
  switch (G) {
    case 1: attention_body<1>(c, d, pre, 1, task); break;
    case 2: attention_body<2>(c, d, pre, 2, task); break;
    default: attention_body<4>(c, d, pre, G, task); break;   // 4 or 8 heads per kv head, four at a time
  }
}

// ---------------------------------------------------------------------------
// TASK_ATTENTION, general instantiation (many requests): per-warp K/V streams through shared memory, tensor-core math
// ---------------------------------------------------------------------------
// With many requests a worker gets whole (request, kv head) pairs or large chunks of them, and what matters is
// bytes in flight and instructions per byte.  The cached positions of the chunk are split evenly over the eight
// compute warps; every warp runs its OWN cp.async pipeline over its share -- steps of 8 positions (K and V rows,
// 4 KB) through a private ring of shared-memory stages, no block-wide barrier inside the loop -- and starts it
// before the task waits for this layer's qkv projection, because rows already in the cache do not depend on it.
// Per step: S = Q K^T on mma.sync m16n8k16 (the query heads of the kv head are the M rows, at most 8 of 16), online
// softmax on the score fragment (fp32, base 2), P rounded to bf16 as the reference does
// (tasks/blackwell/attention_sm100.cuh:558), O += P V on m16n8k8 with V read through ldmatrix.trans.  The rows this
// step appends form one more tile in the same layout, taken by the last warp.  Page ids of the chunk are fetched
// once into shared memory; a step never straddles a page (page sizes are multiples of 8).
constexpr int kAsStepRows = 8;
constexpr int kAsPitch = 272;                              // bytes between rows of a K or V tile (256 + 16: conflict-free ldmatrix)
constexpr int kAsStepBytes = 2 * kAsStepRows * kAsPitch;   // K rows, then V rows
constexpr int kAsPageCap = 256;                            // page ids of a chunk kept in shared memory

struct AttnStream {
  ReqView rv;
  int start, end, new_start, old_end, n_active, nstg, pg0, new_rows_cap;
  int w_begin, w_end;   // cached positions this warp streams
  int issued;           // steps of this warp requested so far
  uint2 cs0, sn0;
  int *pg;              // shared: page ids of pages pg0 .. of the request
  uint8_t *stages;      // shared: [8 warps][nstg] steps
  uint8_t *q_tile;      // shared: 8 rows x kAsPitch, bf16 query heads (rows >= G are zero)
  float *w_ml;          // shared: per warp and head {max, sum}
  uint8_t *new_tile;    // shared: rows appended by this task, K rows then V rows, kAsPitch apart
  // descriptor fields the copy loop needs, read once
  const uint8_t *kbase, *vbase;
  int page, hkv, head, flags, slot, cseq;
};

__device__ __forceinline__ void mma_bf16_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_addr));
}

// This warp requests step `step` of its share (8 positions): a row is 16 pieces of 16 bytes, lane -> piece lane % 16
// of rows lane / 16 + 2 i.  One commit per call, empty or not: the waits count groups.
__device__ __forceinline__ void attn_stream_issue(const Ctx &c, const AttnStream &a, int step, int warp, int lane) {
  const int pos0 = a.w_begin + step * kAsStepRows;
  if (pos0 < a.w_end) {
    size_t off;
    if (a.flags & 4) {
      off = (((size_t)a.slot * a.cseq + pos0) * a.hkv + a.head) * 256;
    } else {
      const int pidx = pos0 / a.page, rel = pidx - a.pg0;
      const int pid = rel < kAsPageCap ? a.pg[rel] : __ldcg(&c.P.meta.paged_kv_indices[a.rv.kv0 + pidx]);
      off = (((size_t)pid * a.page + (pos0 - pidx * a.page)) * a.hkv + a.head) * 256;
    }
    const size_t row_stride = (size_t)a.hkv * 256;
    const int piece = lane & 15, r0 = lane >> 4;
    uint8_t *stage = a.stages + (size_t)(warp * a.nstg + step % a.nstg) * kAsStepBytes;
    const int n = a.w_end - pos0;   // valid rows of this step (>= 1)
#pragma unroll
    for (int i = 0; i < kAsStepRows / 2; ++i) {
      const int r = r0 + 2 * i;
      uint8_t *dst = stage + r * kAsPitch + piece * 16;
      if (r < n) {
        const size_t o = off + (size_t)r * row_stride + piece * 16;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(a.kbase + o) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst + kAsStepRows * kAsPitch)), "l"(a.vbase + o)
                     : "memory");
      } else {
        // positions past the end: defined zeros (a masked position has weight 0, and 0 x NaN from stale bytes would
        // still be NaN in the P V product)
        *reinterpret_cast<uint4 *>(dst) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4 *>(dst + kAsStepRows * kAsPitch) = make_uint4(0, 0, 0, 0);
      }
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

__device__ __forceinline__ void attn_stream_wait(int nstg) {   // all but the (nstg - 2) newest groups have landed
  if (nstg >= 4) asm volatile("cp.async.wait_group 2;" ::: "memory");
  else if (nstg == 3) asm volatile("cp.async.wait_group 1;" ::: "memory");
  else asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Runs before the dependency wait (the batch description is already final): request view, chunk bounds, page ids,
// shared-memory plan, and the first copies of every warp.
template <bool GENERAL>
__device__ __forceinline__ void attention_stream_begin(const Ctx &c, const TaskDesc &d, AttnStream &a, int task) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const volatile int *st = attention_stash<GENERAL>(c, task);
  bool hit = st[0] == task;
  if (hit) {
    a.rv.q0 = st[1]; a.rv.nq = st[2]; a.rv.kv0 = st[3]; a.rv.seq_len = st[4];
    __threadfence_block();
    hit = st[0] == task;
  }
  if (!hit) a.rv = request_view(P, d);
  const int NC = d.a[A_NCHUNK], G = d.a[A_HQ] / d.a[A_HKV];
  a.kbase = reinterpret_cast<const uint8_t *>(d.p[1]);
  a.vbase = reinterpret_cast<const uint8_t *>(d.p[2]);
  a.page = max(d.a[A_PAGE], 1); a.hkv = d.a[A_HKV]; a.head = d.a[A_HEAD]; a.flags = d.a[A_FLAGS];
  a.slot = d.a[A_SLOT]; a.cseq = d.a[A_CSEQ];
  int L = (a.rv.seq_len + NC - 1) / NC;
  L = max((L + 15) & ~15, 16);
  a.n_active = a.rv.nq > 0 ? (a.rv.seq_len + L - 1) / L : 0;
  a.start = d.a[A_CHUNK] * L;
  a.end = min(a.rv.seq_len, a.start + L);
  a.new_start = a.rv.seq_len - a.rv.nq;
  a.old_end = min(a.end, a.new_start);
  const int n_old = (a.rv.nq > 0 && a.old_end > a.start) ? a.old_end - a.start : 0;
  const int per_warp = ((n_old + 7) / 8 + kAsStepRows - 1) / kAsStepRows * kAsStepRows;   // multiple of 8 positions
  a.w_begin = a.start + warp * per_warp;
  a.w_end = min(a.w_begin + per_warp, a.start + n_old);
  a.issued = 0;
  a.cs0 = a.sn0 = make_uint2(0, 0);
  // shared-memory plan: [q tile | warp maxima and sums | page ids | tile of the new rows | stages of the 8 warps]; the
  // per-warp partial outputs of the final combine reuse the stage area once every warp's stream has drained
  uint8_t *base = c.s.xtile;
  a.q_tile = base;
  a.w_ml = reinterpret_cast<float *>(base + 8 * kAsPitch);
  a.pg = reinterpret_cast<int *>(a.w_ml + 8 * G * 2);
  a.new_tile = reinterpret_cast<uint8_t *>(a.pg + kAsPageCap);
  a.new_rows_cap = (min(P.max_num_batched_tokens, 64) + 7) & ~7;
  a.stages = a.new_tile + (size_t)2 * a.new_rows_cap * kAsPitch;
  const int avail = P.x_tile_bytes + kPartialBytes - (int)(a.stages - base);
  a.nstg = max(1, min(4, avail / (8 * kAsStepBytes)));   // (the graph compiler sizes the region for at least two)
  a.pg0 = a.start / a.page;
  if (a.rv.nq <= 0) return;
  load_rope((a.flags & 2) ? reinterpret_cast<const __nv_bfloat16 *>(d.p[5]) : nullptr,
            reinterpret_cast<const __nv_bfloat16 *>(d.p[6]), a.new_start, d.a[A_ROPE_ROWS], lane, a.cs0, a.sn0);
  if (!(a.flags & 4) && n_old > 0) {
    const int n_pg = min((a.old_end - 1) / a.page - a.pg0 + 1, kAsPageCap);
    for (int i = tid; i < n_pg; i += kConsumerThreads) a.pg[i] = __ldcg(&P.meta.paged_kv_indices[a.rv.kv0 + a.pg0 + i]);
  }
  // query rows the kv head does not have stay zero for the whole task; so do the rows of the new-row tile that this
  // step does not fill (masked, but read by the P V product)
  for (int i = tid; i < 8 * kAsPitch / 16; i += kConsumerThreads) reinterpret_cast<uint4 *>(a.q_tile)[i] = make_uint4(0, 0, 0, 0);
  for (int i = tid; i < 2 * a.new_rows_cap * kAsPitch / 16; i += kConsumerThreads)
    reinterpret_cast<uint4 *>(a.new_tile)[i] = make_uint4(0, 0, 0, 0);
  consumer_sync();
  for (int j = 0; j < a.nstg - 1; ++j) attn_stream_issue(c, a, j, warp, lane);
  a.issued = a.nstg - 1;
}

// Eight positions against the query fragments: scores, online softmax, P V.  `n_valid` (1..8): positions below this
// index take part.  The M rows are the query heads (rows 8-15 of the fragments are zero and never read back).
__device__ __forceinline__ void attn_step_mma(const uint8_t *ktile, const uint8_t *vtile, int n_valid, const uint32_t (&qa)[8][2],
                                              float &m_run, float &l_run, float (&o)[16][4], int lane) {
  const int q = lane & 3;
  float sc[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t k_addr = smem_u32(ktile) + (uint32_t)((lane & 7) * kAsPitch + (lane >> 3) * 16);
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    uint32_t b[4];
    ldmatrix_x4(b, k_addr + kk * 64u);
    const uint32_t a0[4] = {qa[2 * kk][0], 0u, qa[2 * kk][1], 0u}, a1[4] = {qa[2 * kk + 1][0], 0u, qa[2 * kk + 1][1], 0u};
    mma_bf16_16816(sc, a0, b[0], b[1]);
    mma_bf16_16816(sc, a1, b[2], b[3]);
  }
  const float qscale = 0.08838834764831845f * 1.4426950408889634f;   // 1/sqrt(128) * log2(e)
  const int col = 2 * q;
  const float s0 = (col < n_valid) ? sc[0] * qscale : -INFINITY;
  const float s1 = (col + 1 < n_valid) ? sc[1] * qscale : -INFINITY;
  float mx = fmaxf(s0, s1);
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  const float mn = fmaxf(m_run, mx);                    // finite: position 0 of the step is valid
  const float corr = exp2f(m_run - mn);                 // 0 on the first step (m_run = -inf)
  const float p0 = exp2f(s0 - mn), p1 = exp2f(s1 - mn);
  float ps = p0 + p1;
  ps += __shfl_xor_sync(0xffffffffu, ps, 1);
  ps += __shfl_xor_sync(0xffffffffu, ps, 2);
  l_run = l_run * corr + ps;
  m_run = mn;
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) { o[nt][0] *= corr; o[nt][1] *= corr; }
  const uint32_t pa = pack_bf16(p0, p1);
  const uint32_t v_addr = smem_u32(vtile) + (uint32_t)((lane & 7) * kAsPitch + (lane >> 3) * 16);
#pragma unroll
  for (int vq = 0; vq < 4; ++vq) {
    uint32_t b[4];
    ldmatrix_x4_trans(b, v_addr + vq * 64u);
#pragma unroll
    for (int i = 0; i < 4; ++i) mma_bf16_1688(o[4 * vq + i], pa, 0u, b[i]);
  }
}

__device__ void attention_stream_body(const Ctx &c, const TaskDesc &d, AttnStream &a, int task) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const ReqView rv = a.rv;
  if (rv.nq <= 0) return;
  const int G = d.a[A_HQ] / d.a[A_HKV];
  const int NC = d.a[A_NCHUNK], chunk = d.a[A_CHUNK], head = d.a[A_HEAD];
  const int hq = d.a[A_HQ];
  const int flags = d.a[A_FLAGS];
  const float eps = __int_as_float(d.a[A_EPS]);
  const __nv_bfloat16 *qkv = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  __nv_bfloat16 *kc = reinterpret_cast<__nv_bfloat16 *>(d.p[1]);
  __nv_bfloat16 *vc = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  const __nv_bfloat16 *qn = (flags & 1) ? reinterpret_cast<const __nv_bfloat16 *>(d.p[3]) : nullptr;
  const __nv_bfloat16 *kn = (flags & 1) ? reinterpret_cast<const __nv_bfloat16 *>(d.p[4]) : nullptr;
  const __nv_bfloat16 *cosT = (flags & 2) ? reinterpret_cast<const __nv_bfloat16 *>(d.p[5]) : nullptr;
  const __nv_bfloat16 *sinT = (flags & 2) ? reinterpret_cast<const __nv_bfloat16 *>(d.p[6]) : nullptr;
  __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[7]);
  const int ldq = d.a[A_LDQKV], ldo = d.a[A_LDO];
  const int rope_rows = d.a[A_ROPE_ROWS];
  const int start = a.start, end = a.end, new_start = a.new_start, n_active = a.n_active;
  const size_t head_base = (size_t)head * (G + 2) * 128;
  float *w_ml = a.w_ml;
  float *w_o = reinterpret_cast<float *>(a.stages);   // [8 warps][G][128], valid once every warp's stream has drained
  uint8_t *new_k = a.new_tile, *new_v = a.new_tile + (size_t)a.new_rows_cap * kAsPitch;
  const int new_lo = max(start, new_start);            // first position this task appends (if any: new_lo < end)
  const bool aprof = P.profiler != nullptr && (uint64_t)(task + 1) * 8 <= P.profiler_entries && tid == 0;

  // ---- append the new keys / values that fall into this chunk (cache + a tile in shared memory) ----
  for (int pos = new_lo + warp; pos < end; pos += 8) {
    const int tok = rv.q0 + (pos - new_start);
    const __nv_bfloat16 *kp = qkv + (size_t)tok * ldq + head_base + (size_t)G * 128 + lane * 4;
    const uint2 kr = __ldcg(reinterpret_cast<const uint2 *>(kp));
    const uint2 vr = __ldcg(reinterpret_cast<const uint2 *>(kp + 128));
    float x[4] = {bf16_lo(kr.x), bf16_hi(kr.x), bf16_lo(kr.y), bf16_hi(kr.y)};
    uint2 cs = a.cs0, sn = a.sn0;
    if (pos != new_start) load_rope(cosT, sinT, pos, rope_rows, lane, cs, sn);
    norm_rope_head(x, kn, eps, cosT != nullptr, cs, sn, lane);
    const uint2 kw = make_uint2(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]));
    const size_t off = kv_offset(P, d, rv, pos) + lane * 4;
    *reinterpret_cast<uint2 *>(kc + off) = kw;
    *reinterpret_cast<uint2 *>(vc + off) = vr;
    const int r = pos - new_lo;
    if (r < a.new_rows_cap) {
      *reinterpret_cast<uint2 *>(new_k + (size_t)r * kAsPitch + lane * 8) = kw;
      *reinterpret_cast<uint2 *>(new_v + (size_t)r * kAsPitch + lane * 8) = vr;
    }
  }
  const int g = lane >> 2, q = lane & 3;
  const int my_steps = a.w_end > a.w_begin ? (a.w_end - a.w_begin + kAsStepRows - 1) / kAsStepRows : 0;
  bool first_pass = true;                    // the copies of the first pass were started before the dependency wait

  for (int t = 0; t < rv.nq; ++t) {
    const int pq = new_start + t;
    const int tok = rv.q0 + t;
    const int lim = min(end, pq + 1);
    if (t > 0) consumer_sync();              // the combine of the previous token has read the stage area
    if (warp < G) {
      const __nv_bfloat16 *qp = qkv + (size_t)tok * ldq + head_base + (size_t)warp * 128 + lane * 4;
      const uint2 qr = __ldcg(reinterpret_cast<const uint2 *>(qp));
      float x[4] = {bf16_lo(qr.x), bf16_hi(qr.x), bf16_lo(qr.y), bf16_hi(qr.y)};
      uint2 cs = a.cs0, sn = a.sn0;
      if (t != 0) load_rope(cosT, sinT, pq, rope_rows, lane, cs, sn);
      norm_rope_head(x, qn, eps, cosT != nullptr, cs, sn, lane);   // (results are bf16-rounded values)
      *reinterpret_cast<uint2 *>(a.q_tile + (size_t)warp * kAsPitch + lane * 8) =
          make_uint2(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]));
    }
    consumer_sync();   // the q tile and the tile of new rows are ready
    if (aprof && t == 0) P.profiler[(size_t)task * 8 + 4] = globaltimer_ns();
    uint32_t qa[8][2];   // rows 0-7 of the A fragments of the eight k steps (rows 8-15 are zero)
    {
      const uint32_t q_addr = smem_u32(a.q_tile) + (uint32_t)((lane & 7) * kAsPitch + ((lane >> 3) & 1) * 16);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) ldmatrix_x2(qa[ks], q_addr + ks * 32u);
    }
    float m_run = -INFINITY, l_run = 0.f;
    float o[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    // ---- this warp's share of the cached rows, step by step through its own stage ring ----
    if (!first_pass) {
      for (int j = 0; j < a.nstg - 1; ++j) attn_stream_issue(c, a, j, warp, lane);
      a.issued = a.nstg - 1;
    }
    first_pass = false;
    for (int j = 0; j < my_steps; ++j) {
      attn_stream_wait(a.nstg);
      __syncwarp();                                      // step j has landed for the whole warp; stage (j - 1) % nstg is free
      attn_stream_issue(c, a, j + a.nstg - 1, warp, lane);
      if (a.nstg == 1) {   // a single stage cannot run ahead: the step just requested is the one consumed now
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
      }
      const uint8_t *stg = a.stages + (size_t)(warp * a.nstg + j % a.nstg) * kAsStepBytes;
      attn_step_mma(stg, stg + kAsStepRows * kAsPitch, min(kAsStepRows, a.w_end - (a.w_begin + j * kAsStepRows)), qa, m_run, l_run, o,
                    lane);
      __syncwarp();                                      // every lane is done reading the stage before it is refilled
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (aprof && t == 0) P.profiler[(size_t)task * 8 + 5] = globaltimer_ns();
    // ---- rows appended by this task (causal: query token t sees the new rows up to its own position): last warp ----
    if (warp == 7 && new_lo < lim) {
      const int n_new = min(lim - new_lo, a.new_rows_cap);
      for (int r0 = 0; r0 < n_new; r0 += kAsStepRows)
        attn_step_mma(new_k + (size_t)r0 * kAsPitch, new_v + (size_t)r0 * kAsPitch, min(kAsStepRows, n_new - r0), qa, m_run, l_run, o,
                      lane);
    }
    consumer_sync();   // every warp's stream has drained: the stage area becomes the partial-output area
    if (g < G) {
      float *wo = &w_o[((size_t)warp * G + g) * 128 + 2 * q];
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) *reinterpret_cast<float2 *>(wo + nt * 8) = make_float2(o[nt][0], o[nt][1]);
      if (q == 0) {
        w_ml[(warp * G + g) * 2 + 0] = m_run;
        w_ml[(warp * G + g) * 2 + 1] = l_run;
      }
    }
    consumer_sync();
    if (aprof && t == 0) P.profiler[(size_t)task * 8 + 6] = globaltimer_ns();
    // combine the 8 warps; thread -> (g, dim) pairs
    for (int idx = tid; idx < G * 128; idx += kConsumerThreads) {
      const int gg = idx >> 7, dd = idx & 127;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 8; ++w) M = fmaxf(M, w_ml[(w * G + gg) * 2]);
      float Ls = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float mw = w_ml[(w * G + gg) * 2];
        const float scw = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
        Ls += w_ml[(w * G + gg) * 2 + 1] * scw;
        O += w_o[((size_t)w * G + gg) * 128 + dd] * scw;
      }
      const int hq_idx = head * G + gg;
      if (NC == 1) {
        out[(size_t)tok * ldo + (size_t)hq_idx * 128 + dd] = __float2bfloat16_rn(Ls > 0.f ? O / Ls : 0.f);
      } else {
        const size_t base = ((size_t)tok * hq + hq_idx) * NC + chunk;
        __stcg(&P.attn_scratch[base * 130 + 2 + dd], O);
        if (dd == 0) {
          __stcg(&P.attn_scratch[base * 130 + 0], M);
          __stcg(&P.attn_scratch[base * 130 + 1], Ls);
        }
      }
    }
  }
  if (NC == 1) return;
  // ---- split-KV merge by the last chunk task to arrive ---------------------------
  consumer_sync();
  if (tid == 0) {
    unsigned int old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;"
                 : "=r"(old)
                 : "l"(&P.attn_tickets[d.a[A_TICKET] + d.a[A_SLOT] * d.a[A_HKV] + head])
                 : "memory");
    c.s.flags[1] = ((old + 1u) % (unsigned)NC == 0u) ? 1 : 0;
  }
  consumer_sync();
  if (c.s.flags[1] == 0) return;
  for (int item = warp; item < rv.nq * G * 4; item += 8) {
    const int row = item >> 2, dd = ((item & 3) << 5) + lane;
    const int t = row / G, gg = row - t * G;
    const int tok = rv.q0 + t;
    const int hq_idx = head * G + gg;
    const size_t base = ((size_t)tok * hq + hq_idx) * NC;
    const bool v = lane < n_active;
    const float m = v ? __ldcg(&P.attn_scratch[(base + lane) * 130]) : -INFINITY;
    const float l = v ? __ldcg(&P.attn_scratch[(base + lane) * 130 + 1]) : 0.f;
    float ow[16], ow2[16];
#pragma unroll
    for (int u = 0; u < 16; ++u)
      ow[u] = (u < n_active) ? __ldcg(&P.attn_scratch[(base + u) * 130 + 2 + dd]) : 0.f;
    if (n_active > 16) {
#pragma unroll
      for (int u = 0; u < 16; ++u)
        ow2[u] = (16 + u < n_active) ? __ldcg(&P.attn_scratch[(base + 16 + u) * 130 + 2 + dd]) : 0.f;
    }
    float M = m;
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o2));
    const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
    const float Ls = warp_sum(l * w);
    float O = 0.f;
#pragma unroll
    for (int u = 0; u < 16; ++u) O = fmaf(ow[u], __shfl_sync(0xffffffffu, w, u), O);
    if (n_active > 16) {
#pragma unroll
      for (int u = 0; u < 16; ++u) O = fmaf(ow2[u], __shfl_sync(0xffffffffu, w, 16 + u), O);
    }
    out[(size_t)tok * ldo + (size_t)hq_idx * 128 + dd] = __float2bfloat16_rn(Ls > 0.f ? O / Ls : 0.f);
  }
}

__device__ __forceinline__ void run_attention_stream(const Ctx &c, const TaskDesc &d, AttnStream &a, int task) {
  attention_stream_body(c, d, a, task);
}

// ---------------------------------------------------------------------------
// small tasks
// ---------------------------------------------------------------------------
__device__ void run_embed(const Ctx &c, const TaskDesc &d) {
  const int B = active_tokens(c.P);
  const int t0 = d.a[E_T0], t1 = min(d.a[E_T1], B), width = d.a[E_WIDTH];
  const int64_t *ids = reinterpret_cast<const int64_t *>(d.p[0]);
  const __nv_bfloat16 *tab = reinterpret_cast<const __nv_bfloat16 *>(d.p[1]);
  __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  const int vecs = width / 8;
  for (int t = t0; t < t1; ++t) {
    const long long id = __ldcg(reinterpret_cast<const long long *>(&ids[t]));
    for (int v = threadIdx.x; v < vecs; v += kConsumerThreads) {
      uint4 val = make_uint4(0, 0, 0, 0);
      // ids outside the table (e.g. the argmax of a row of NaNs) read as a zero row instead of a wild address
      if (id >= 0 && id < (long long)d.a[E_AUX]) val = __ldg(reinterpret_cast<const uint4 *>(tab + (size_t)id * d.a[E_LDI]) + v);
      reinterpret_cast<uint4 *>(out + (size_t)t * d.a[E_LDO])[v] = val;
    }
  }
}

__device__ void run_rmsnorm(const Ctx &c, const TaskDesc &d) {
  const int B = active_tokens(c.P);
  const int t0 = d.a[E_T0], t1 = min(d.a[E_T1], B), width = d.a[E_WIDTH];
  const __nv_bfloat16 *in = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  const __nv_bfloat16 *gam = reinterpret_cast<const __nv_bfloat16 *>(d.p[1]);
  __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  const float eps = __int_as_float(d.a[E_AUX]);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int vecs = width / 8;
  for (int t = t0; t < t1; ++t) {
    const uint4 *row = reinterpret_cast<const uint4 *>(in + (size_t)t * d.a[E_LDI]);
    float ss = 0.f;
    for (int v = tid; v < vecs; v += kConsumerThreads) {
      const uint4 x = __ldcg(row + v);
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) ss += bf16_lo(w[q]) * bf16_lo(w[q]) + bf16_hi(w[q]) * bf16_hi(w[q]);
    }
    ss = warp_sum(ss);
    if (lane == 0) c.s.red[warp] = ss;
    consumer_sync();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += c.s.red[w];
    const float inv = rsqrtf(tot / (float)width + eps);
    for (int v = tid; v < vecs; v += kConsumerThreads) {
      const uint4 x = __ldcg(row + v);
      const uint4 g = __ldg(reinterpret_cast<const uint4 *>(gam) + v);
      const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, gw[4] = {g.x, g.y, g.z, g.w};
      uint32_t ow[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        ow[q] = pack_bf16(bf16_lo(xw[q]) * inv * bf16_lo(gw[q]), bf16_hi(xw[q]) * inv * bf16_hi(gw[q]));
      reinterpret_cast<uint4 *>(out + (size_t)t * d.a[E_LDO])[v] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    consumer_sync();
  }
}

// silu_mul over columns [a[7], a[8]) of the activation (width a[2] = I), group-interleaved input
__device__ void run_silu_mul(const Ctx &c, const TaskDesc &d) {
  const int B = active_tokens(c.P);
  const int t0 = d.a[E_T0], t1 = min(d.a[E_T1], B), I = d.a[E_WIDTH];
  const int groups = d.a[E_AUX];
  const int per = I / groups;
  const __nv_bfloat16 *in = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  const int c0 = d.a[7], c1 = d.a[8];
  if (((per | c0 | c1 | d.a[E_LDI] | d.a[E_LDO]) & 7) == 0 && ((d.p[0] | d.p[2]) & 15) == 0 && t1 > t0) {
    // 16-byte vectors (eight columns of one interleave group), tokens and columns flattened over the threads so that
    // every thread has several independent loads in flight
    const int nv = (c1 - c0) >> 3, total = nv * (t1 - t0);
    for (int i = threadIdx.x; i < total; i += kConsumerThreads) {
      const int t = t0 + i / nv, j = c0 + ((i - (i / nv) * nv) << 3);
      const int g = j / per, off = j - g * per;
      const __nv_bfloat16 *gp = in + (size_t)t * d.a[E_LDI] + (size_t)g * 2 * per + off;
      const uint4 gv = __ldcg(reinterpret_cast<const uint4 *>(gp));
      const uint4 uv = __ldcg(reinterpret_cast<const uint4 *>(gp + per));
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
      uint32_t ow[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float g0 = bf16_lo(gw[q]), g1 = bf16_hi(gw[q]);
        const float a0 = round_bf16(g0 / (1.0f + expf(-g0))), a1 = round_bf16(g1 / (1.0f + expf(-g1)));
        ow[q] = pack_bf16(a0 * bf16_lo(uw[q]), a1 * bf16_hi(uw[q]));
      }
      *reinterpret_cast<uint4 *>(out + (size_t)t * d.a[E_LDO] + j) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    return;
  }
  for (int t = t0; t < t1; ++t)
    for (int j = c0 + threadIdx.x; j < c1; j += kConsumerThreads) {
      const int g = j / per, off = j - g * per;
      const float gv = bf16_to_f(__ldcg(&in[(size_t)t * d.a[E_LDI] + (size_t)g * 2 * per + off]));
      const float uv = bf16_to_f(__ldcg(&in[(size_t)t * d.a[E_LDI] + (size_t)g * 2 * per + per + off]));
      const float a = round_bf16(gv / (1.0f + expf(-gv)));
      out[(size_t)t * d.a[E_LDO] + j] = __float2bfloat16_rn(a * uv);
    }
}

__device__ void run_elementwise_add(const Ctx &c, const TaskDesc &d) {
  const int B = active_tokens(c.P);
  const int t0 = d.a[E_T0], t1 = min(d.a[E_T1], B), width = d.a[E_WIDTH];
  const __nv_bfloat16 *a = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  const __nv_bfloat16 *b = reinterpret_cast<const __nv_bfloat16 *>(d.p[1]);
  __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  for (int t = t0; t < t1; ++t)
    for (int j = threadIdx.x; j < width; j += kConsumerThreads)
      out[(size_t)t * d.a[E_LDO] + j] = __float2bfloat16_rn(bf16_to_f(__ldcg(&a[(size_t)t * d.a[E_LDI] + j])) +
                                                           bf16_to_f(__ldcg(&b[(size_t)t * d.a[E_LDI2] + j])));
}

__device__ void run_tensor_init(const Ctx &c, const TaskDesc &d) {
  // zero rows [t0,t1) of width a[2] BYTES
  uint8_t *out = reinterpret_cast<uint8_t *>(d.p[2]);
  const size_t row_bytes = (size_t)d.a[E_WIDTH];
  for (int t = d.a[E_T0]; t < d.a[E_T1]; ++t)
    for (size_t j = threadIdx.x * 4; j < row_bytes; j += kConsumerThreads * 4)
      *reinterpret_cast<uint32_t *>(out + (size_t)t * d.a[E_LDO] + j) = 0u;
}

// (value, index) argmax with lowest-index tie-break
__device__ __forceinline__ void argmax_merge(float &v, long long &i, float v2, long long i2) {
  if (v2 > v || (v2 == v && i2 < i)) {
    v = v2;
    i = i2;
  }
}

__device__ void block_argmax(const Ctx &c, float &v, long long &i) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
    const long long i2 = __shfl_xor_sync(0xffffffffu, i, o);
    argmax_merge(v, i, v2, i2);
  }
  long long *ri = reinterpret_cast<long long *>(c.s.red + 16);
  if (lane == 0) {
    c.s.red[warp] = v;
    ri[warp] = i;
  }
  consumer_sync();
  v = c.s.red[0];
  i = ri[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) argmax_merge(v, i, c.s.red[w], ri[w]);
  consumer_sync();
}

// ---- Gumbel-max sampling (the reference's sampling task, tasks/common/sampling.cuh:100-226) --------------------
// Philox4x32-10 as cuRAND's curand_init(seed, subsequence, offset 0) followed by one curand_uniform4 uses it: the
// counter is (0, 0, subsequence low, subsequence high), the key is the seed, and the four outputs map to
// (0, 1] by x * 2^-32 + 2^-33.
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += 0x9E3779B9u;
    key.y += 0xBB67AE85u;
  }
  return ctr;
}

__device__ __forceinline__ float gumbel_noise(uint32_t r) {
  const float u = fmaf(__uint2float_rn(r), 2.3283064e-10f, 1.1641532e-10f);
  return -0.6931471806f * __log2f(-__log2f(u + 1e-20f) + 1e-20f);
}

// (value, index) maximum where equal values go to the highest index: the order the reference's block reduction
// resolves ties in (later element, higher lane, later warp, later pass).
__device__ __forceinline__ void sample_merge(float &v, long long &i, float v2, long long i2) {
  if (v2 > v || (v2 == v && i2 > i)) {
    v = v2;
    i = i2;
  }
}

// One column range of the vocabulary: key = bf16(logit + bf16(noise)), noise by groups of four columns from one
// Philox block whose subsequence is (row within the reference task) * V + first column of the group.
__device__ void run_sampling_partial(const Ctx &c, const TaskDesc &d) {
  const int B = active_tokens(c.P);
  const __nv_bfloat16 *logits = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  __nv_bfloat16 *pv = reinterpret_cast<__nv_bfloat16 *>(d.p[1]);
  long long *pi = reinterpret_cast<long long *>(d.p[2]);
  const int c0 = d.a[0], c1 = d.a[1], cid = d.a[2], ldl = d.a[3], ldp = d.a[4];
  const uint2 key = make_uint2((uint32_t)d.a[6], (uint32_t)d.a[7]);
  const int rows_per_task = max(d.a[8], 1);
  const uint32_t V = (uint32_t)d.a[9];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  long long *ri = reinterpret_cast<long long *>(c.s.red + 16);
  for (int b = 0; b < B; ++b) {
    float v = -INFINITY;
    long long i = -1;
    const uint32_t row_base = (uint32_t)(b % rows_per_task) * V;
    for (int q = (c0 >> 2) + tid; q * 4 < c1; q += kConsumerThreads) {
      const uint4 r = philox4x32_10(make_uint4(0u, 0u, row_base + (uint32_t)q * 4u, 0u), key);
      const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = q * 4 + e;
        if (j >= c0 && j < c1) {
          const float noise = bf16_to_f(__float2bfloat16_rn(gumbel_noise(rr[e])));
          const float k = bf16_to_f(__float2bfloat16_rn(bf16_to_f(__ldcg(&logits[(size_t)b * ldl + j])) + noise));
          sample_merge(v, i, k, (long long)j);
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
      const long long i2 = __shfl_xor_sync(0xffffffffu, i, o);
      sample_merge(v, i, v2, i2);
    }
    if (lane == 0) {
      c.s.red[warp] = v;
      ri[warp] = i;
    }
    consumer_sync();
    if (tid == 0) {
      for (int w = 1; w < 8; ++w) sample_merge(v, i, c.s.red[w], ri[w]);
      pv[(size_t)b * ldp + cid] = __float2bfloat16_rn(v);
      pi[(size_t)b * ldp + cid] = i;
    }
    consumer_sync();
  }
}

__device__ void run_sampling_reduce(const Ctx &c, const TaskDesc &d) {
  const int B = active_tokens(c.P);
  const __nv_bfloat16 *pv = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  const long long *pi = reinterpret_cast<const long long *>(d.p[1]);
  long long *out = reinterpret_cast<long long *>(d.p[2]);
  const int n = d.a[0], ldp = d.a[1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int b = warp; b < B; b += 8) {
    float v = -INFINITY;
    long long i = -1;
    for (int j = lane; j < n; j += 32)
      sample_merge(v, i, bf16_to_f(__ldcg(&pv[(size_t)b * ldp + j])), __ldcg(&pi[(size_t)b * ldp + j]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
      const long long i2 = __shfl_xor_sync(0xffffffffu, i, o);
      sample_merge(v, i, v2, i2);
    }
    if (lane == 0) out[b] = i < 0 ? 0 : i;
  }
}

__device__ void run_argmax_partial(const Ctx &c, const TaskDesc &d) {
  const int B = active_tokens(c.P);
  const __nv_bfloat16 *logits = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  __nv_bfloat16 *pv = reinterpret_cast<__nv_bfloat16 *>(d.p[1]);
  long long *pi = reinterpret_cast<long long *>(d.p[2]);
  const int c0 = d.a[0], c1 = d.a[1], cid = d.a[2], ldl = d.a[3], ldp = d.a[4];
  for (int b = 0; b < B; ++b) {
    float v = -INFINITY;
    long long i = 0x7fffffffffffffffLL;
    for (int j = c0 + threadIdx.x; j < c1; j += kConsumerThreads)
      argmax_merge(v, i, bf16_to_f(__ldcg(&logits[(size_t)b * ldl + j])), (long long)j);
    block_argmax(c, v, i);
    if (threadIdx.x == 0) {
      pv[(size_t)b * ldp + cid] = __float2bfloat16_rn(v);
      pi[(size_t)b * ldp + cid] = i;
    }
  }
}

__device__ void run_argmax_reduce(const Ctx &c, const TaskDesc &d) {
  const int B = active_tokens(c.P);
  const __nv_bfloat16 *pv = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  const long long *pi = reinterpret_cast<const long long *>(d.p[1]);
  long long *out = reinterpret_cast<long long *>(d.p[2]);
  const int n = d.a[0], ldp = d.a[1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int b = warp; b < B; b += 8) {
    float v = -INFINITY;
    long long i = 0x7fffffffffffffffLL;
    for (int j = lane; j < n; j += 32)
      argmax_merge(v, i, bf16_to_f(__ldcg(&pv[(size_t)b * ldp + j])), __ldcg(&pi[(size_t)b * ldp + j]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
      const long long i2 = __shfl_xor_sync(0xffffffffu, i, o);
      argmax_merge(v, i, v2, i2);
    }
    if (lane == 0) out[b] = i;
  }
}

// Argmax over a vocabulary sharded across the ranks.  Warp b merges this rank's partials of token b, then lane r
// exchanges with rank r: it stores this rank's {value | seq} and {index | seq} 64-bit words into rank r's inbox and
// polls, in its own inbox, for the pair rank r pushed; the warp then takes the best pair (largest value, lowest index).
// Every rank sees the same pairs and writes the same id.
__device__ __forceinline__ void run_argmax_exchange(const Ctx &c, const TaskDesc &d) {
  const KernelParams &P = c.P;
  const int B = active_tokens(P);
  const __nv_bfloat16 *pv = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  const long long *pi = reinterpret_cast<const long long *>(d.p[1]);
  long long *out = reinterpret_cast<long long *>(d.p[2]);
  const int n = d.a[0], ldp = d.a[1], W = P.world_size, mbt = P.max_num_batched_tokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned long long inst = c.iteration * (unsigned)d.a[L_NAR] + (unsigned)d.a[L_ARIDX];
  const unsigned long long seq = (unsigned long long)ll_seq(c.iteration, d.a[L_NAR], d.a[L_ARIDX]);
  const size_t area = (size_t)d.p[5] + (size_t)(inst & 1ull) * (size_t)d.a[L_PARSTRIDE];   // in 32-bit words
  for (int b = warp; b < B; b += 8) {
    float v = -INFINITY;
    long long i = 0x7fffffffffffffffLL;
    for (int j = lane; j < n; j += 32)
      argmax_merge(v, i, bf16_to_f(__ldcg(&pv[(size_t)b * ldp + j])), __ldcg(&pi[(size_t)b * ldp + j]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
      const long long i2 = __shfl_xor_sync(0xffffffffu, i, o);
      argmax_merge(v, i, v2, i2);
    }
    i += (long long)d.a[2];   // column of the whole vocabulary (all lanes hold the merged pair)
    float rv = -INFINITY;
    long long ri = 0x7fffffffffffffffLL;
    if (lane < W) {
      const size_t slot = ((size_t)P.rank * mbt + b) * 4;
      unsigned long long *dst = reinterpret_cast<unsigned long long *>(reinterpret_cast<uint32_t *>(P.peer_inbox[lane]) + area + slot);
      const unsigned long long w0 = (unsigned long long)__float_as_uint(v) | (seq << 32);
      const unsigned long long w1 = ((unsigned long long)i & 0xffffffffull) | (seq << 32);
      asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(dst), "l"(w0), "l"(w1) : "memory");
      const unsigned long long *src = reinterpret_cast<const unsigned long long *>(
          reinterpret_cast<const uint32_t *>(P.peer_inbox[P.rank]) + area + ((size_t)lane * mbt + b) * 4);
      uint32_t polls = 0;
      while (true) {
        unsigned long long a0, a1;
        asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a0), "=l"(a1) : "l"(src) : "memory");
        if ((a0 >> 32) == seq && (a1 >> 32) == seq) {
          rv = __uint_as_float((uint32_t)a0);
          ri = (long long)(a1 & 0xffffffffull);
          break;
        }
        if ((++polls & 0xff) == 0) {
          if (ld_volatile_i32(&P.status->error) != 0) break;
          if (globaltimer_ns() > c.deadline_ns) {
            report_timeout(P.status, c.worker, 3, lane);
            break;
          }
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float v2 = __shfl_xor_sync(0xffffffffu, rv, o);
      const long long i2 = __shfl_xor_sync(0xffffffffu, ri, o);
      argmax_merge(rv, ri, v2, i2);
    }
    if (lane == 0) out[b] = ri;
  }
}

// Sum the per-rank fp32 inbox slots in rank order (+ residual) -> bf16.
__device__ void run_allreduce(const Ctx &c, const TaskDesc &d) {
  const KernelParams &P = c.P;
  const int B = active_tokens(P);
  const int c0 = d.a[0], c1 = d.a[1], world = d.a[2], slot = d.a[3], ldo = d.a[4], ldr = d.a[5], N = d.a[6];
  const size_t parity = (size_t)((c.iteration * (unsigned)d.a[8] + (unsigned)d.a[7]) & 1ull);
  const float *inbox = P.peer_inbox[P.rank] + (size_t)d.p[0] + parity * (size_t)d.a[9];
  const __nv_bfloat16 *res = reinterpret_cast<const __nv_bfloat16 *>(d.p[1]);
  __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(d.p[2]);
  const int w = c1 - c0;
  for (int idx = threadIdx.x; idx < B * w; idx += kConsumerThreads) {
    const int b = idx / w, j = c0 + (idx - b * w);
    float v = 0.f;
    for (int r = 0; r < world; ++r) v += __ldcg(&inbox[(size_t)r * slot + (size_t)b * N + j]);
    if (res) v += bf16_to_f(__ldcg(&res[(size_t)b * ldr + j]));
    out[(size_t)b * ldo + j] = __float2bfloat16_rn(v);
  }
}

// Push stage of an unfused allreduce: columns [c0, c1) of a local bf16 tensor go, as fp32, into this rank's slot of
// every rank's inbox; the task's event is incremented on every rank once the stores are ordered (TF_REMOTE_TRIGGER).
__device__ void run_ar_push(const Ctx &c, const TaskDesc &d) {
  const KernelParams &P = c.P;
  const int B = active_tokens(P);
  const int c0 = d.a[0], c1 = d.a[1], ldx = d.a[2], slot = d.a[3], N = d.a[6];
  const size_t parity = (size_t)((c.iteration * (unsigned)d.a[8] + (unsigned)d.a[7]) & 1ull);
  const size_t base = (size_t)d.p[5] + parity * (size_t)d.a[9] + (size_t)P.rank * (size_t)slot;
  const __nv_bfloat16 *x = reinterpret_cast<const __nv_bfloat16 *>(d.p[0]);
  const int w = c1 - c0;
  for (int idx = threadIdx.x; idx < B * w; idx += kConsumerThreads) {
    const int b = idx / w, j = c0 + (idx - b * w);
    const float v = bf16_to_f(__ldcg(&x[(size_t)b * ldx + j]));
    for (int peer = 0; peer < P.world_size; ++peer) P.peer_inbox[peer][base + (size_t)b * N + j] = v;
  }
}

// ---------------------------------------------------------------------------
// TASK_BATCH: device-side continuous batching, block-parallel.
// Same result, array by array, as the reference's single-threaded
// prepare_next_batch (include/mirage/persistent_kernel/persistent_kernel.cuh:206-368).
// ---------------------------------------------------------------------------
__device__ __noinline__ void run_batch(const Ctx c) {
  if (c.tmem_base & 0x80000000u) {   // called for TASK_ARGMAX_EXCHANGE (see task_other)
    run_argmax_exchange(c, c.s.desc[c.tmem_base & 1u]);
    return;
  }
  const KernelParams &P = c.P;
  const BatchMeta &M = P.meta;
  const int tid = threadIdx.x;
  const int mbr = P.max_num_batched_requests, mbt = P.max_num_batched_tokens;
  const int PS = P.page_size, S = P.max_seq_length, MP = P.max_num_pages;
  int *sm = reinterpret_cast<int *>(c.s.xtile);
  int *s_rid = sm;                 // [mbr]  request id per old slot (-1 when empty or retired)
  int *s_kv = s_rid + mbr;         // [mbr+1] old kv indptr
  int *s_step = s_kv + mbr + 1;    // [mbr]  updated step
  int *s_plen = s_step + mbr;      // [mbr]
  int *s_free = s_plen + mbr;      // [mbr+1] pages freed (then exclusive prefix)
  int *n_rid = s_free + mbr + 1;   // [mbr]  new slot -> request id
  int *n_tok = n_rid + mbr;        // [mbr+1] new qo indptr
  int *n_pg = n_tok + mbr + 1;     // [mbr+1] new kv indptr
  int *n_old = n_pg + mbr + 1;     // [mbr]  pages carried over
  int *n_src = n_old + mbr;        // [mbr]  old kv offset of carried pages
  int *n_newoff = n_src + mbr;     // [mbr]  offset into freshly allocated pages
  int *n_step = n_newoff + mbr;    // [mbr]  token read offset in `tokens`
  int *sc = n_step + mbr;          // scalars: [0] head [1] tail [2] next_req [3] num_reqs [4] num_tokens [5] num_pages

  const int prev_tokens = M.qo_indptr[mbr];   // active tokens of the previous iteration (0 after a reset)
  if (tid < 3) sc[tid] = M.sched_scalars[tid];
  for (int i = tid; i <= mbr; i += kConsumerThreads) s_kv[i] = M.paged_kv_indptr[i];
  consumer_sync();
  // Step 1: commit outputs, advance steps, retire finished requests.
  // s_rid: request id, -1 for an empty slot, -2 for a request retired in this step.
  for (int i = tid; i < mbr; i += kConsumerThreads) {
    int rid = M.request_ids[i];
    int freed = 0, step_new = 0, plen = 0;
    if (rid != -1) {
      const int step = M.step[rid];
      const int qo = M.qo_indptr[i];
      const int n = M.qo_indptr[i + 1] - qo;
      plen = M.prompt_lengths[rid];
      for (int j = 0; j < n; ++j)
        if (step + j + 1 >= plen && step + j + 1 < S)
          M.tokens[(size_t)rid * S + step + j + 1] = M.output_tokens[qo + j];
      step_new = step + n;
      M.step[rid] = step_new;
      const bool done = (step_new + 1 >= S) ||
                        (M.tokens[(size_t)rid * S + step_new] == P.eos_token_id && step_new >= plen);
      if (done) {
        freed = s_kv[i + 1] - s_kv[i];
        rid = -2;
      }
    }
    s_free[i] = freed;
    s_rid[i] = rid;
    s_step[i] = step_new;
    s_plen[i] = plen;
  }
  consumer_sync();
  if (tid == 0) {
    int acc = 0;
    for (int i = 0; i < mbr; ++i) {
      const int f = s_free[i];
      s_free[i] = acc;
      acc += f;
    }
    s_free[mbr] = acc;
  }
  consumer_sync();
  for (int i = 0; i < mbr; ++i) {
    if (s_rid[i] != -2) continue;
    const int cnt = s_free[i + 1] - s_free[i];
    for (int j = tid; j < cnt; j += kConsumerThreads)
      M.page_queue[(unsigned)(sc[1] + s_free[i] + j) % (unsigned)MP] = M.paged_kv_indices[s_kv[i] + j];
  }
  // Step 2: snapshot of the page table (compaction below may overlap its source).
  for (int i = tid; i < s_kv[mbr]; i += kConsumerThreads) M.paged_kv_indices_snapshot[i] = M.paged_kv_indices[i];
  consumer_sync();
  // Step 3: lay out the next batch (serial over slots, all operands in shared memory).
  if (tid == 0) {
    int num_reqs = 0, num_tokens = 0, num_pages = 0, new_pages = 0;
    int head = sc[0];
    for (int i = 0; i < mbr; ++i) {
      const int rid = s_rid[i];
      if (rid < 0) continue;
      const int step = s_step[i];
      int nn = s_plen[i] - step;
      nn = (nn > 0) ? min(nn, mbt - num_tokens) : min(1, mbt - num_tokens);
      const int n_old_pages = s_kv[i + 1] - s_kv[i];
      const int np = (step + nn + PS - 1) / PS;
      n_rid[num_reqs] = rid;
      n_tok[num_reqs] = num_tokens;
      n_pg[num_reqs] = num_pages;
      n_old[num_reqs] = n_old_pages;
      n_src[num_reqs] = s_kv[i];
      n_newoff[num_reqs] = new_pages;
      n_step[num_reqs] = step;
      new_pages += max(np - n_old_pages, 0);
      num_pages += np;
      num_tokens += nn;
      ++num_reqs;
    }
    int next = sc[2];
    while (num_reqs < mbr && num_tokens < mbt && next < P.total_num_requests) {
      const int nn = min(M.prompt_lengths[next], mbt - num_tokens);
      const int np = (nn + PS - 1) / PS;
      n_rid[num_reqs] = next;
      n_tok[num_reqs] = num_tokens;
      n_pg[num_reqs] = num_pages;
      n_old[num_reqs] = 0;
      n_src[num_reqs] = 0;
      n_newoff[num_reqs] = new_pages;
      n_step[num_reqs] = 0;
      new_pages += np;
      num_pages += np;
      num_tokens += nn;
      ++num_reqs;
      ++next;
    }
    n_tok[num_reqs] = num_tokens;
    n_pg[num_reqs] = num_pages;
    sc[3] = num_reqs;
    sc[4] = num_tokens;
    sc[5] = num_pages;
    sc[6] = head;              // ring position of the first fresh page
    sc[0] = head + new_pages;
    sc[1] = sc[1] + s_free[mbr];
    sc[2] = next;
  }
  consumer_sync();
  const int num_reqs = sc[3], num_tokens = sc[4], num_pages = sc[5], head0 = sc[6];
  // Step 4: write the batch description.
  for (int k = 0; k < num_reqs; ++k) {
    const int rid = n_rid[k];
    const int nn = n_tok[k + 1] - n_tok[k];
    const int np = n_pg[k + 1] - n_pg[k];
    for (int j = tid; j < nn; j += kConsumerThreads)
      M.input_tokens[n_tok[k] + j] = M.tokens[(size_t)rid * S + n_step[k] + j];
    for (int j = tid; j < np; j += kConsumerThreads) {
      int pg;
      if (j < n_old[k]) pg = M.paged_kv_indices_snapshot[n_src[k] + j];
      else pg = M.page_queue[(unsigned)(head0 + n_newoff[k] + (j - n_old[k])) % (unsigned)MP];
      M.paged_kv_indices[n_pg[k] + j] = pg;
    }
  }
  for (int k = tid; k < mbr; k += kConsumerThreads) {
    if (k < num_reqs) {
      M.request_ids[k] = n_rid[k];
      M.qo_indptr[k] = n_tok[k];
      M.paged_kv_indptr[k] = n_pg[k];
      const int tot = n_step[k] + (n_tok[k + 1] - n_tok[k]);
      const int lpl = tot % PS;
      M.paged_kv_last_page_len[k] = (lpl == 0) ? PS : lpl;
    } else {
      M.request_ids[k] = -1;
      M.qo_indptr[k] = num_tokens;
      M.paged_kv_indptr[k] = num_pages;
    }
  }
  if (P.world_size > 1 && P.ll_row_words > 0 && num_tokens < prev_tokens) {
    // token rows that go idle: no sequence number may survive in them (see ll_seq)
    uint32_t *inbox = reinterpret_cast<uint32_t *>(P.peer_inbox[P.rank]);
    const size_t N = (size_t)P.ll_row_words, span = (size_t)(prev_tokens - num_tokens) * N;
    for (int buf = 0; buf < 2; ++buf)
      for (int r = 0; r < P.world_size; ++r) {
        uint32_t *rows = inbox + (size_t)buf * (size_t)P.ll_buffer_words + ((size_t)r * mbt + (size_t)num_tokens) * N;
        for (size_t i = tid; i < span; i += kConsumerThreads) rows[i] = 0u;
      }
  }
  if (tid == 0) {
    M.qo_indptr[mbr] = num_tokens;
    M.paged_kv_indptr[mbr] = num_pages;
    M.sched_scalars[0] = sc[0];
    M.sched_scalars[1] = sc[1];
    M.sched_scalars[2] = sc[2];
    P.status->active_tokens = num_tokens;
    P.status->all_done = (num_tokens == 0) ? 1 : 0;
  }
}

// ---------------------------------------------------------------------------
// compute warps: walk the task list
// ---------------------------------------------------------------------------
struct TaskTimes {   // profiler timestamps of the running task (thread 0 only)
  uint64_t begin_ns, ready_ns;
  bool on;
};

// Thread 0 acquire-polls the task's event counters, then the compute warps meet.  Returns false when
// the launch is being abandoned.
__device__ __forceinline__ bool wait_dependencies(const Ctx &c, const TaskDesc &d, int t, bool ok, TaskTimes &tt) {
  const KernelParams &P = c.P;
  if (threadIdx.x == 0) {
    if (tt.on) tt.begin_ns = globaltimer_ns();
    bool good = ok;
    for (int i = 0; i < kMaxDeps && good; ++i) {
      const int ev = d.dep_event[i];
      if (ev < 0) continue;
      good = wait_counter(c, &P.counters[ev], (unsigned long long)d.dep_need[i] * c.iteration,
                          (d.flags & (TF_DEP0_REMOTE << i)) != 0, 1, t);
    }
    if (!good) c.s.flags[0] = 1;
    if (tt.on) tt.ready_ns = globaltimer_ns();
  }
  consumer_sync();
  return c.s.flags[0] == 0;
}

// Each task kind has its own non-inlined runner so that register allocation of the heavy bodies
// (attention) does not leak into the weight-streaming loop.
template <bool GENERAL, bool TPX>
__device__ __forceinline__ bool task_linear(const Ctx &c, const TaskDesc &d, int t, bool ok, TaskTimes &tt,
                                         LinearState &ls) {
  const int tid = threadIdx.x;
  // constants the prologue needs are fetched before the dependency wait
  uint4 gpre[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
  if (d.a[L_PRO] == PRO_RMSNORM) {
    const uint4 *gam = reinterpret_cast<const uint4 *>(d.p[4]);
    const int vecs = d.a[L_KT] / 8;
    if (tid < vecs) gpre[0] = __ldg(gam + tid);
    if (tid + kConsumerThreads < vecs) gpre[1] = __ldg(gam + tid + kConsumerThreads);
  }
  ok = wait_dependencies(c, d, t, ok, tt);
  // the weight chunks must be consumed even when the launch is being abandoned or no token is active
  if (GENERAL && (d.flags & TF_TC) && (d.flags & TF_FP8)) run_linear_fp8_tc(c, d, ls, t, ok);
  else if (GENERAL && (d.flags & TF_TC)) run_linear_tc(c, d, ls, t, gpre, ok);
  else if (GENERAL && (d.flags & TF_FP8)) run_linear_fp8(c, d, ls, t, ok);
  else run_linear<GENERAL, TPX>(c, d, ls, t, gpre, ok);
  return ok;
}

template <bool GENERAL>
__device__ __forceinline__ bool task_attention(const Ctx &c, const TaskDesc &d, int t, bool ok, TaskTimes &tt) {
  const KernelParams &P = c.P;
  // the batch description must be final before the page table is read; that event fired long ago
  if (d.a[A_EARLY_EV] >= 0) {
    if (threadIdx.x == 0 && ok &&
        !wait_counter(c, &P.counters[d.a[A_EARLY_EV]], (unsigned long long)d.a[A_EARLY_NEED] * c.iteration,
                      false, 1, t))
      c.s.flags[0] = 1;
    consumer_sync();
    ok = ok && (c.s.flags[0] == 0);
  }
  if (GENERAL) {
    AttnStream as;
    as.rv.nq = 0;
    if (tt.on && threadIdx.x == 0) P.profiler[(size_t)t * 8 + 7] = globaltimer_ns();
    if (ok) attention_stream_begin<GENERAL>(c, d, as, t);
    ok = wait_dependencies(c, d, t, ok, tt);
    if (ok) run_attention_stream(c, d, as, t);
    asm volatile("cp.async.wait_group 0;" ::: "memory");   // (also on the abandoned path: nothing may stay in flight)
    return ok;
  }
  AttnPre pre;
  pre.rv.nq = 0;
  if (ok) attention_prefetch<GENERAL>(c, d, pre, t);
  if (threadIdx.x == 0) *reinterpret_cast<volatile int *>(&c.s.flags[2]) = 1;   // quiet the weight stream
  ok = wait_dependencies(c, d, t, ok, tt);
  if (ok) run_attention(c, d, pre, t);
  if (threadIdx.x == 0) *reinterpret_cast<volatile int *>(&c.s.flags[2]) = 0;
  return ok;
}

template <bool GENERAL, bool TPX>
__device__ __forceinline__ bool task_other(const Ctx &c, const TaskDesc &d, int t, bool ok, TaskTimes &tt) {
  ok = wait_dependencies(c, d, t, ok, tt);
  if (!ok) return false;
  switch (d.type) {
    // (the argmax exchange of multi-rank graphs shares the batching task's out-of-line function and its call site: a
    // second call in this switch moved the register allocation of the linear loop; bit 31 of the tensor-memory field,
    // never set in an address, says which body is meant and which descriptor slot holds the task)
    case TASK_ARGMAX_EXCHANGE: if (!TPX) break; [[fallthrough]];
    case TASK_BATCH: {
      Ctx cc = c;
      if (TPX && d.type == TASK_ARGMAX_EXCHANGE) cc.tmem_base = 0x80000000u | (&d == &c.s.desc[1] ? 1u : 0u);
      run_batch(cc);
      break;
    }
    case TASK_EMBED: run_embed(c, d); break;
    case TASK_RMSNORM: run_rmsnorm(c, d); break;
    case TASK_SILU_MUL: run_silu_mul(c, d); break;
    case TASK_ARGMAX_PARTIAL: run_argmax_partial(c, d); break;
    case TASK_ARGMAX_REDUCE: run_argmax_reduce(c, d); break;
    case TASK_ALLREDUCE: run_allreduce(c, d); break;
    case TASK_ELEMENTWISE_ADD: run_elementwise_add(c, d); break;
    case TASK_TENSOR_INIT: run_tensor_init(c, d); break;
    case TASK_QUANTIZE_FP8: if (GENERAL) run_quantize_fp8(c, d); break;
    case TASK_MOE_ROUTING: if (GENERAL) run_moe_routing(c, d); break;
    case TASK_MOE_SILU_MUL: if (GENERAL) run_moe_silu_mul(c, d); break;
    case TASK_MOE_MUL_SUM_ADD: if (GENERAL) run_moe_mul_sum_add(c, d); break;
    case TASK_MLA_APPEND: if (GENERAL) run_mla_append(c, d); break;
    case TASK_MLA_DECODE: if (GENERAL) run_mla_decode(c, d); break;
    case TASK_MLA_REDUCE: if (GENERAL) run_mla_reduce(c, d); break;
    case TASK_SAMPLING_PARTIAL: if (GENERAL) run_sampling_partial(c, d); break;
    case TASK_SAMPLING_REDUCE: if (GENERAL) run_sampling_reduce(c, d); break;
    case TASK_AR_PUSH: if (GENERAL && TPX) run_ar_push(c, d); break;
    default: break;
  }
  return true;
}

template <bool GENERAL, bool TPX>
__device__ void consumer_loop(const Ctx &c, int t_begin, int t_end) {
  const KernelParams &P = c.P;
  const int tid = threadIdx.x;
  LinearState ls{0, 0u, 0u};
  if (t_begin < t_end && tid < kDescVecs)
    reinterpret_cast<uint4 *>(&c.s.desc[0])[tid] = __ldg(reinterpret_cast<const uint4 *>(&P.tasks[t_begin]) + tid);
  consumer_sync();
  bool ok = true;
  for (int t = t_begin; t < t_end; ++t) {
    const TaskDesc &d = c.s.desc[(t - t_begin) & 1];
    uint4 nxt = make_uint4(0, 0, 0, 0);
    const bool fetch = (t + 1 < t_end) && tid >= 224 && tid < 224 + kDescVecs;
    if (fetch) nxt = __ldg(reinterpret_cast<const uint4 *>(&P.tasks[t + 1]) + (tid - 224));
    TaskTimes tt{0, 0, (P.profiler != nullptr) && (uint64_t)(t + 1) * 8 <= P.profiler_entries};
    const uint32_t type = d.type;
    if (type == TASK_LINEAR) ok = task_linear<GENERAL, TPX>(c, d, t, ok, tt, ls);
    else if (GENERAL && type == TASK_MOE_GEMM) {
      ok = wait_dependencies(c, d, t, ok, tt);
      run_moe_gemm(c, d, ls, t, ok);
    } else if (type == TASK_ATTENTION) ok = task_attention<GENERAL>(c, d, t, ok, tt);
    else ok = task_other<GENERAL, TPX>(c, d, t, ok, tt);
    if (fetch) reinterpret_cast<uint4 *>(&c.s.desc[(t + 1 - t_begin) & 1])[tid - 224] = nxt;
    const int trig = d.trig_event;
    const uint32_t tflags = d.flags;
    consumer_sync();
    ok = ok && (c.s.flags[0] == 0);
    if (!ok) break;
    if (tid == 0 && tt.on) {
      // per task: [wait begin, dependencies satisfied, body end, worker << 40 | event << 8 | type]  (globaltimer ns)
      uint64_t *rec = P.profiler + (size_t)t * 8;
      rec[0] = tt.begin_ns;
      rec[1] = tt.ready_ns;
      rec[2] = globaltimer_ns();
      rec[3] = ((uint64_t)c.worker << 40) | ((uint64_t)(uint32_t)trig << 8) | (uint64_t)type;
    }
    if (tid == 0 && trig >= 0) {
      // red.release orders this CTA's writes (observed through the barrier above) before the increment
      if (tflags & TF_REMOTE_TRIGGER) {
        // one system-scope fence orders the pushed partial sums before the counter increments; the increments
        // themselves are relaxed so that they travel to all peers concurrently instead of one round trip each
        __threadfence_system();
        for (int r = 0; r < P.world_size; ++r) red_relaxed_sys(&P.peer_counters[r][trig], 1ull);
      } else {
        red_release_gpu(&P.counters[trig], 1ull);
      }
    }
  }
}

// Two instantiations: GENERAL = false is the batch-1 product path (bf16 weights, at most 8 batched tokens),
// kept free of every other task body so that its register allocation at the 168-register cap stays as tuned;
// GENERAL = true adds FP8 tasks and linear tasks for up to 64 tokens.  The host picks by graph content.
// TPX marks the instantiations that graphs of more than one rank run.  Code written for tensor parallelism after the
// single-GPU paths had been tuned sits behind it -- the allreduce prologue with all ranks' loads in flight (batch-1
// kernel), the argmax exchange of a sharded lm_head -- so that the single-GPU instantiations <*, false> stay exactly
// the code that was measured: both run at the register cap, where unrelated code moves their allocation.
template <bool GENERAL, bool TPX = false>
__global__ void __launch_bounds__(kBlockThreads, 1) mpk_megakernel(const __grid_constant__ KernelParams P) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  Smem s = carve(smem_raw, P);
  const int tid = threadIdx.x;
  const unsigned long long iteration = *reinterpret_cast<volatile unsigned long long *>(&P.status->iteration) + 1ull;
  if (tid == 0) {
    if (blockIdx.x == 0) P.status->t_start[iteration & 7] = globaltimer_ns();
    for (int i = 0; i < P.num_stages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 8);
    }
    s.flags[0] = 0;
    s.flags[1] = 0;
    s.flags[2] = 0;
    *reinterpret_cast<volatile int *>(&s.full[8]) = -1;   // attention stash: empty
    if (GENERAL)
      for (int i = 0; i < kStashRing; ++i) reinterpret_cast<volatile int *>(s.flags + 16)[i * 8] = -1;
    if (GENERAL) mbar_init(s.acc_bar, 8);   // one tcgen05.commit per compute warp
    mbar_fence_init();
  }
  // graphs with tcgen05 tasks: warp 0 takes all 512 tensor-memory columns (one CTA per SM, so nothing else asks)
  const bool use_tmem = GENERAL && P.use_tmem != 0;
  if (use_tmem && tid < 32) tmem_alloc(s.tmem_holder, kTmemCols);
  if (use_tmem) tc_fence_before_sync();
  __syncthreads();
  if (use_tmem) tc_fence_after_sync();
  Ctx c{P, s, iteration, globaltimer_ns() + (uint64_t)P.spin_limit * 1000000ull, (int)blockIdx.x,
        use_tmem ? *reinterpret_cast<volatile uint32_t *>(s.tmem_holder) : 0u};
  const int t_begin = P.worker_begin[blockIdx.x], t_end = P.worker_begin[blockIdx.x + 1];
  if (tid >= kConsumerThreads) {
    streamer_loop<GENERAL>(c, t_begin, t_end);
  } else {
    consumer_loop<GENERAL, TPX>(c, t_begin, t_end);
  }
  if (use_tmem) tc_fence_before_sync();
  __syncthreads();
  if (use_tmem && tid < 32) {
    // Every exit path of both loops ends here.  MMAs still in flight after an abandoned launch must finish before
    // the columns are freed: one more commit, awaited with a bounded number of polls.
    tc_fence_after_sync();
    if (tid == 0 && s.flags[0] != 0) {
      // parity is unknown after an abort: a fresh barrier in the (now idle) full-barrier array
      mbar_init(&s.full[15], 1);
      mbar_fence_init();
      umma_commit(&s.full[15]);
      uint32_t polls = 0;
      while (!mbar_try_wait(&s.full[15], 0u) && ++polls < (1u << 22)) {}
    }
    __syncwarp();
    tmem_dealloc(c.tmem_base, kTmemCols);
  }
  if (tid == 0) {
    __threadfence();
    const unsigned int ticket = atomicAdd(&P.status->exit_ticket, 1u);
    if (ticket == gridDim.x - 1) {
      P.status->exit_ticket = 0;
      P.status->t_end[iteration & 7] = globaltimer_ns();
      P.status->iteration = iteration;
      __threadfence();
    }
  }
}

}  // namespace mpk

// ---------------------------------------------------------------------------
// host-side launch glue (called from the C ABI implementation)
// ---------------------------------------------------------------------------
extern "C" int mpk_kernel_smem_bytes(int num_stages, int stage_bytes, int x_tile_bytes) {
  return num_stages * stage_bytes + x_tile_bytes + mpk::kPartialBytes + mpk::kMiscBytes;
}

// The limit is a property of the function on the current device, shared by every handle of the process: it is raised
// to the device's opt-in maximum (not to this handle's need), so that preparing a graph with a small footprint cannot
// lower it under a graph prepared earlier.
extern "C" int mpk_kernel_prepare(int smem_bytes) {
  int dev = 0, limit = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (e != cudaSuccess) return (int)e;
  if (smem_bytes > limit) return (int)cudaErrorInvalidValue;
  smem_bytes = limit;
  e = cudaFuncSetAttribute(mpk::mpk_megakernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(mpk::mpk_megakernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(mpk::mpk_megakernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(mpk::mpk_megakernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int mpk_kernel_launch(const mpk::KernelParams *params, int smem_bytes, void *stream) {
  if (params->general_kernel && params->world_size > 1)
    mpk::mpk_megakernel<true, true><<<params->num_workers, mpk::kBlockThreads, smem_bytes, (cudaStream_t)stream>>>(*params);
  else if (params->general_kernel)
    mpk::mpk_megakernel<true><<<params->num_workers, mpk::kBlockThreads, smem_bytes, (cudaStream_t)stream>>>(*params);
  else if (params->world_size > 1 && params->tp_extensions)
    mpk::mpk_megakernel<false, true><<<params->num_workers, mpk::kBlockThreads, smem_bytes, (cudaStream_t)stream>>>(*params);
  else
    mpk::mpk_megakernel<false><<<params->num_workers, mpk::kBlockThreads, smem_bytes, (cudaStream_t)stream>>>(*params);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

__global__ void mpk_shuffle_rows_kernel(uint8_t *dst, const uint8_t *const *srcs, const int64_t *rows_per_group,
                                        const int64_t *prefix_rows, int n, int64_t group_rows_total,
                                        int64_t row_bytes, int64_t total_rows) {
  // dst row r: group g = r / group_rows_total, offset o within the group; tensor i with prefix[i] <= o < prefix[i+1]
  for (int64_t r = blockIdx.x; r < total_rows; r += gridDim.x) {
    const int64_t g = r / group_rows_total, o = r - g * group_rows_total;
    int i = 0;
    while (i + 1 < n && o >= prefix_rows[i + 1]) ++i;
    const uint8_t *src = srcs[i] + ((g * rows_per_group[i]) + (o - prefix_rows[i])) * row_bytes;
    uint8_t *d = dst + r * row_bytes;
    if (row_bytes % 16 == 0) {
      for (int64_t b = threadIdx.x * 16; b < row_bytes; b += blockDim.x * 16)
        *reinterpret_cast<uint4 *>(d + b) = *reinterpret_cast<const uint4 *>(src + b);
    } else {   // narrow rows (e.g. the packed scale words of a small weight): 4-byte words
      for (int64_t b = threadIdx.x * 4; b < row_bytes; b += blockDim.x * 4)
        *reinterpret_cast<uint32_t *>(d + b) = *reinterpret_cast<const uint32_t *>(src + b);
    }
  }
}

extern "C" int mpk_shuffle_rows_launch(void *dst, const void *const *srcs_dev, const int64_t *rows_per_group_dev,
                                       const int64_t *prefix_rows_dev, int n, int64_t group_rows_total,
                                       int64_t row_bytes, int64_t total_rows, void *stream) {
  mpk_shuffle_rows_kernel<<<1024, 256, 0, (cudaStream_t)stream>>>(
      (uint8_t *)dst, (const uint8_t *const *)srcs_dev, rows_per_group_dev, prefix_rows_dev, n, group_rows_total,
      row_bytes, total_rows);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}
