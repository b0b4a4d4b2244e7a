// Fused data-parallel step over NVLink peer memory: gradient reduce-scatter + unscale +
// non-finite agreement + partitioned AdamW + all-gather of the updated 16-bit weights, in ONE
// kernel per rank (one process per GPU; every rank launches the same kernel on its own stream).
//
// Every rank owns a contiguous shard of the flat parameter space.  Its kernel
//   1. waits until every rank has finished its backward (flag barrier over peer memory),
//   2. reads its shard of the fp32 gradient bucket from EVERY rank with plain P2P vector loads
//      (the loads of all peers are issued before any is consumed), sums them into its own
//      bucket and notes whether anything was non-finite,
//   3. (dynamic loss scaling only) publishes its non-finite flag to all ranks and barriers, so
//      that all ranks take the same skip decision; a decision agreed outside the kernel, over
//      a whole PPxDP job, is passed in instead and costs no barrier,
//   4. applies Adam/AdamW on the shard, all optimizer groups in one launch, with moments that
//      exist only on the owner (ZeRO-1 memory), and writes the new 16-bit weights into EVERY
//      rank's shadow buffer with P2P vector stores.  The fp32 masters stay with the owner; only
//      the tail of each group that some op reads in fp32 (biases, norm weights: `master_from`)
//      is pushed to the peers' master buffers,
//   5. barriers again so nobody starts the next forward on half-written weights, and clears the
//      part of its own gradient bucket that other ranks own (they have all read it by then).
// Bytes over NVLink per parameter: 4 read + 2 written, times (world-1)/world.
// No NCCL call, no TMA and no multicast load is involved; all remote traffic is ld/st.global on
// IPC-mapped peer pointers.  Barriers are epoch counters written with st.release.sys and
// polled with ld.acquire.sys.  Every poll is bounded by the run-time wait limit of the status
// buffer; a wait that runs out is STICKY for the call: the kernel records
// PF_ERR_TIMEOUT_PEER_FLAG, marks the step as skipped, touches no weight, no moment and no peer
// memory afterwards, and returns.  The host reads the status word once per step.
#include <cstring>
#include "common.cuh"
#include "api.h"

namespace pf {

constexpr int DP_MAX = 8;
constexpr int DP_MAX_GROUPS = 8;
constexpr int DP_THREADS = 512;
constexpr int DP_CTAS_PER_SM = 2;
// Ranks reach the first barrier of a step with the skew of a whole training step between them
// (first-step compilation, graph capture), so that wait gets this multiple of the limit; the
// later barriers only cover the kernel's own phases.
constexpr int DP_ENTRY_WAIT_FACTOR = 10;

struct DpGroup {
  long long lo, hi;            // range of the flat buffer this optimizer group covers
  long long local_below;       // 16-bit weights below this index are written locally only: their
                               // first consumer gathers the rows other ranks own
  long long master_from;       // fp32 masters at or above this index also go to every peer
  float lr, beta1, beta2, eps, weight_decay;
  int adamw;
};

struct DpArgs {
  int rank, world;
  float* grad[DP_MAX];
  float* master[DP_MAX];
  void* lp[DP_MAX];            // null when there is no 16-bit shadow
  int* flags[DP_MAX];          // per rank: int[DP_MAX] barrier slots + int[DP_MAX] found slots
  float* m;                    // local moments, indexed from shard_lo
  float* v;
  int* local_sync;             // local: [0] arrival counter, [1] release word, [2] failed epoch
  long long shard_lo, shard_hi;
  long long total;             // length of the flat buffers
  int ngroups;
  DpGroup group[DP_MAX_GROUPS];
  float grad_scale;
  int lp_dtype;
  int check_inf;               // 1: agree on non-finite gradients inside the kernel
  int found_given;             // 1: *found_inf already holds the job-wide decision
  const float* loss_scale;     // local device scalar (identical on every rank) or null
  float* found_inf;            // local: 1 when the step was skipped
  const int* applied_steps;    // device counter of optimizer steps that were applied so far
  int host_step;               // used when applied_steps is null
  int epoch;                   // epoch of this call's first barrier (same on every rank)
  int sync_base;               // arrivals at local_sync[0] before this call
  int* status;
  long long* trace;            // optional: nanosecond timestamps of the phases (CTA 0)
};

__device__ __forceinline__ void dp_mark(const DpArgs& a, int slot) {
  if (a.trace && blockIdx.x == 0 && threadIdx.x == 0) {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    a.trace[slot] = t;
  }
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// counters wrap: "a has reached b" in modular arithmetic
__device__ __forceinline__ bool reached(int a, int b) { return (int)((unsigned)a - (unsigned)b) >= 0; }

// All CTAs of this GPU and all ranks meet here.  `k` = ordinal of the barrier within the call.
// Returns false on every thread of every CTA of this GPU when any wait of this call ran out.
__device__ bool job_barrier(const DpArgs& a, int k) {
  __shared__ int s_failed;
  __threadfence_system();
  __syncthreads();
  const int epoch = a.epoch + k;
  if (threadIdx.x == 0) {
    const long long limit = wait_limit(a.status) * (k == 0 ? DP_ENTRY_WAIT_FACTOR : 1);
    const int target = a.sync_base + (k + 1) * (int)gridDim.x;
    atomicAdd(&a.local_sync[0], 1);
    bool ok = true;
    if (blockIdx.x == 0) {
      long long t0 = clock64();
      while (!reached(ld_acquire_gpu(&a.local_sync[0]), target)) {
        if (clock64() - t0 > limit) { ok = false; break; }
      }
      if (ok) {
        __threadfence_system();
        for (int p = 0; p < a.world; ++p) st_release_sys(&a.flags[p][a.rank], epoch);
        for (int r = 0; r < a.world && ok; ++r) {
          t0 = clock64();
          while (!reached(ld_acquire_sys(&a.flags[a.rank][r]), epoch)) {
            if (clock64() - t0 > limit) { ok = false; break; }
          }
        }
      }
      if (!ok) {
        report(a.status, PF_ERR_TIMEOUT_PEER_FLAG);
        atomicExch(&a.local_sync[2], a.epoch);      // sticky for this call
      }
      __threadfence_system();
      atomicExch(&a.local_sync[1], epoch);          // release the other CTAs either way
    } else {
      const long long t0 = clock64();
      while (!reached(ld_acquire_gpu(&a.local_sync[1]), epoch)) {
        if (clock64() - t0 > 2 * limit + limit * a.world) {
          report(a.status, PF_ERR_TIMEOUT_PEER_FLAG);
          atomicExch(&a.local_sync[2], a.epoch);
          break;
        }
      }
    }
    s_failed = ld_acquire_gpu(&a.local_sync[2]) == a.epoch;
  }
  __syncthreads();
  return !s_failed;
}

// Eight consecutive floats of one thread.  With 32-byte alignment they move as one 256-bit
// access, so that a warp touches 1 KB of whole sectors per instruction; two 16-byte accesses
// per lane would leave every instruction with half-used sectors.
struct F8 { float4 a, b; };
__device__ __forceinline__ F8 ld8(const float* p, bool wide) {
  F8 r;
  if (wide) {
    asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.a.x), "=f"(r.a.y), "=f"(r.a.z), "=f"(r.a.w),
                   "=f"(r.b.x), "=f"(r.b.y), "=f"(r.b.z), "=f"(r.b.w)
                 : "l"(p));
  } else {
    r.a = *reinterpret_cast<const float4*>(p);
    r.b = *reinterpret_cast<const float4*>(p + 4);
  }
  return r;
}
__device__ __forceinline__ void st8(float* p, const F8& r, bool wide) {
  if (wide) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::
                 "l"(p), "f"(r.a.x), "f"(r.a.y), "f"(r.a.z), "f"(r.a.w),
                 "f"(r.b.x), "f"(r.b.y), "f"(r.b.z), "f"(r.b.w) : "memory");
  } else {
    *reinterpret_cast<float4*>(p) = r.a;
    *reinterpret_cast<float4*>(p + 4) = r.b;
  }
}

template <int WORLD>
__global__ void __launch_bounds__(DP_THREADS, DP_CTAS_PER_SM)
dp_fused_kernel(const DpArgs a) {
  const long long lo = a.shard_lo, hi = a.shard_hi;
  const long long nvec = (hi - lo) / 4;        // shards are multiples of 4 elements
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  int kbar = 0;

  dp_mark(a, 0);
  bool ok = job_barrier(a, kbar++);            // every rank's gradients are complete
  dp_mark(a, 1);
  if (!ok) { if (tid == 0 && a.found_inf) *a.found_inf = 1.f; return; }

  // ---- reduce-scatter into the local bucket.  One or two 16-byte vectors per thread from each
  //      of the WORLD buckets (128 bytes per thread in all) are requested before any is consumed.
  bool bad = false;
  constexpr int U = WORLD <= 4 ? 2 : 1;
  for (long long i0 = tid; i0 < nvec; i0 += stride * U) {
    float4 g[WORLD][U];
#pragma unroll
    for (int p = 0; p < WORLD; ++p)
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        g[p][u] = i < nvec ? __ldcs(reinterpret_cast<const float4*>(a.grad[p] + lo + i * 4))
                           : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      float4 s = g[0][u];
#pragma unroll
      for (int p = 1; p < WORLD; ++p) {
        s.x += g[p][u].x; s.y += g[p][u].y; s.z += g[p][u].z; s.w += g[p][u].w;
      }
      if (i < nvec) {
        if (WORLD > 1) *reinterpret_cast<float4*>(a.grad[a.rank] + lo + i * 4) = s;
        if (a.check_inf)
          bad |= !(isfinite(s.x) && isfinite(s.y) && isfinite(s.z) && isfinite(s.w));
      }
    }
  }

  dp_mark(a, 2);
  bool skip = false;
  if (a.check_inf) {
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0)
      for (int p = 0; p < a.world; ++p) st_release_sys(&a.flags[p][DP_MAX + a.rank], a.epoch);
    ok = job_barrier(a, kbar++);               // everybody's non-finite flag is published
    if (!ok) { if (tid == 0 && a.found_inf) *a.found_inf = 1.f; return; }
    for (int r = 0; r < a.world; ++r)
      skip |= ld_acquire_sys(&a.flags[a.rank][DP_MAX + r]) == a.epoch;
    if (tid == 0) *a.found_inf = skip ? 1.f : 0.f;
  } else {
    // the update loop below deals the reduced gradients to the threads in another order (eight
    // consecutive elements per thread) than the loop above wrote them: every CTA must have
    // finished its part of the reduce before any thread reads the sums
    ok = job_barrier(a, kbar++);
    if (!ok) { if (tid == 0 && a.found_inf) *a.found_inf = 1.f; return; }
    if (a.found_given) skip = *reinterpret_cast<const volatile float*>(a.found_inf) != 0.f;
  }
  dp_mark(a, 3);
  float gs = a.grad_scale;
  if (a.loss_scale) gs /= *a.loss_scale;
  const float step = (float)(a.applied_steps ? *a.applied_steps + 1 : a.host_step);

  // ---- partitioned Adam/AdamW; new 16-bit weights go to every rank by P2P stores.  A thread
  //      updates 8 consecutive elements, so that every remote store carries 16 bytes (a warp
  //      writes 512 contiguous bytes per peer; 8-byte stores reached a fifth of the link rate).
  int gi = 0;
  float lr = 0.f, b1 = 0.f, b2 = 0.f, eps = 0.f, wd = 0.f, inv_bc1 = 1.f, inv_sqrt_bc2 = 1.f;
  bool adamw = true;
  long long g_lo = 0, g_hi = -1, local_below = 0, master_from = 0;
  const long long nvec8 = (hi - lo) / 8;       // whole 8-element groups; a 4-element tail follows
  const long long n_items = nvec8 + (((hi - lo) & 7) ? 1 : 0);
  // 256-bit accesses need 32-byte alignment of every stream at element e (and of m, v at i * 8)
  const bool wide = ((lo & 7) == 0) &&
      (((reinterpret_cast<uintptr_t>(a.grad[a.rank]) | reinterpret_cast<uintptr_t>(a.master[a.rank]) |
         reinterpret_cast<uintptr_t>(a.m) | reinterpret_cast<uintptr_t>(a.v)) & 31) == 0);
  const F8 z8 = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  for (long long i = tid; i < n_items; i += stride) {
    const long long e = lo + i * 8;
    const bool two = i < nvec8;                // false: the trailing 4 elements of the shard
    F8 g8 = z8, w8 = z8, m8 = z8, v8 = z8;
    if (two) {
      g8 = ld8(a.grad[a.rank] + e, wide);
      if (!skip) {
        w8 = ld8(a.master[a.rank] + e, wide);
        m8 = ld8(a.m + i * 8, wide);
        v8 = ld8(a.v + i * 8, wide);
      }
      st8(a.grad[a.rank] + e, z8, wide);
    } else {
      g8.a = *reinterpret_cast<const float4*>(a.grad[a.rank] + e);
      if (!skip) {
        w8.a = *reinterpret_cast<const float4*>(a.master[a.rank] + e);
        m8.a = *reinterpret_cast<const float4*>(a.m + i * 8);
        v8.a = *reinterpret_cast<const float4*>(a.v + i * 8);
      }
      *reinterpret_cast<float4*>(a.grad[a.rank] + e) = z8.a;
    }
    if (skip) continue;
    if (e < g_lo || e >= g_hi) {               // entered another optimizer group
      for (gi = 0; gi < a.ngroups - 1 && !(e >= a.group[gi].lo && e < a.group[gi].hi); ++gi) {}
      const DpGroup& G = a.group[gi];
      g_lo = G.lo; g_hi = G.hi; local_below = G.local_below; master_from = G.master_from;
      lr = G.lr; b1 = G.beta1; b2 = G.beta2; eps = G.eps; wd = G.weight_decay;
      adamw = G.adamw != 0;
      inv_bc1 = 1.f / (1.f - powf(b1, step));
      inv_sqrt_bc2 = rsqrtf(1.f - powf(b2, step));
    }
    float g[8] = {g8.a.x, g8.a.y, g8.a.z, g8.a.w, g8.b.x, g8.b.y, g8.b.z, g8.b.w};
    float w[8] = {w8.a.x, w8.a.y, w8.a.z, w8.a.w, w8.b.x, w8.b.y, w8.b.z, w8.b.w};
    float m[8] = {m8.a.x, m8.a.y, m8.a.z, m8.a.w, m8.b.x, m8.b.y, m8.b.z, m8.b.w};
    float v[8] = {v8.a.x, v8.a.y, v8.a.z, v8.a.w, v8.b.x, v8.b.y, v8.b.z, v8.b.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {              // (the upper four are zeros in the 4-element tail)
      float gr = g[j] * gs;
      if (adamw) w[j] *= (1.f - lr * wd);
      else gr += wd * w[j];
      m[j] = b1 * m[j] + (1.f - b1) * gr;
      v[j] = b2 * v[j] + (1.f - b2) * gr * gr;
      w[j] -= lr * (m[j] * inv_bc1) / (sqrtf(v[j]) * inv_sqrt_bc2 + eps);
    }
    w8.a = make_float4(w[0], w[1], w[2], w[3]); w8.b = make_float4(w[4], w[5], w[6], w[7]);
    m8.a = make_float4(m[0], m[1], m[2], m[3]); m8.b = make_float4(m[4], m[5], m[6], m[7]);
    v8.a = make_float4(v[0], v[1], v[2], v[3]); v8.b = make_float4(v[4], v[5], v[6], v[7]);
    uint32_t q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (a.lp_dtype == PF_BF16) {
        __nv_bfloat162 x = __floats2bfloat162_rn(w[2 * j], w[2 * j + 1]);
        q[j] = *reinterpret_cast<uint32_t*>(&x);
      } else {
        __half2 x = __floats2half2_rn(w[2 * j], w[2 * j + 1]);
        q[j] = *reinterpret_cast<uint32_t*>(&x);
      }
    }
    // group boundaries are multiples of 128 elements and shards of 4: an 8-element group never
    // straddles a group, and its two halves share the push decisions
    const bool push_lp = e >= local_below, push_master = e >= master_from;
    if (two) {
      st8(a.m + i * 8, m8, wide);
      st8(a.v + i * 8, v8, wide);
      st8(a.master[a.rank] + e, w8, wide);
      const uint4 q8 = make_uint4(q[0], q[1], q[2], q[3]);
      if (a.lp[a.rank])
        *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(a.lp[a.rank]) + e) = q8;
#pragma unroll
      for (int p = 0; p < WORLD; ++p) {
        if (p == a.rank) continue;
        if (push_master) {
          *reinterpret_cast<float4*>(a.master[p] + e) = w8.a;
          *reinterpret_cast<float4*>(a.master[p] + e + 4) = w8.b;
        }
        if (a.lp[p] && push_lp)
          *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(a.lp[p]) + e) = q8;
      }
    } else {
      *reinterpret_cast<float4*>(a.m + i * 8) = m8.a;
      *reinterpret_cast<float4*>(a.v + i * 8) = v8.a;
      *reinterpret_cast<float4*>(a.master[a.rank] + e) = w8.a;
      const uint2 q4 = make_uint2(q[0], q[1]);
      if (a.lp[a.rank])
        *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(a.lp[a.rank]) + e) = q4;
#pragma unroll
      for (int p = 0; p < WORLD; ++p) {
        if (p == a.rank) continue;
        if (push_master) *reinterpret_cast<float4*>(a.master[p] + e) = w8.a;
        if (a.lp[p] && push_lp)
          *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(a.lp[p]) + e) = q4;
      }
    }
  }

  dp_mark(a, 4);
  ok = job_barrier(a, kbar++);                  // all weights have landed everywhere
  if (!ok) return;
  dp_mark(a, 5);

  // ---- every rank has read what it needed of this bucket: clear the part of it that other
  //      ranks own (local stores; the own shard was cleared by the update loop)
  {
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const long long n_before = lo / 4, n_after = (a.total - hi) / 4;
    for (long long i = tid; i < n_before; i += stride)
      *reinterpret_cast<float4*>(a.grad[a.rank] + i * 4) = z4;
    for (long long i = tid; i < n_after; i += stride)
      *reinterpret_cast<float4*>(a.grad[a.rank] + hi + i * 4) = z4;
  }
  dp_mark(a, 6);
}

}  // namespace pf

using namespace pf;

// Pointer tables are arrays of `world` device pointers (entry `rank` is the local buffer).
// [shard_lo, shard_hi) is the part of the flat buffers [0, total) that this rank owns: it
// reduces and updates its shard and clears the whole of its own gradient bucket.
// `groups` holds `ngroups` records of 4 long long (lo, hi, local_below, master_from) and
// `hyper` `ngroups` records of 6 floats (lr, beta1, beta2, eps, weight_decay, adamw != 0).
// `epoch` is the value of this call's first barrier: it must be identical on every rank and
// grow by the number of barriers a call uses (3), which the call returns
// through *barriers_out; `arrivals_before` is the sum over earlier calls of barriers * grid
// (*grid_out).  `applied_steps` (device int, may be null) counts the optimizer steps that were
// not skipped; the bias correction uses it, so a step skipped on an overflow does not count.
// `trace` (device int64[7], may be null) receives the global-timer value in nanoseconds when CTA 0
// enters the kernel, leaves the entry barrier, finishes its share of the reduce, knows the skip
// decision, finishes its share of the update, leaves the last barrier, and finishes clearing.
PF_API int pf_dp_fused_step(int rank, int world, void* const* grad, void* const* master,
                            void* const* lp, void* const* flags, void* m, void* v,
                            void* local_sync, long long shard_lo, long long shard_hi,
                            long long total, int ngroups, const long long* groups,
                            const float* hyper, const void* applied_steps, int host_step,
                            float grad_scale, int lp_dtype, int check_inf, int found_given,
                            const void* loss_scale, void* found_inf, int epoch,
                            int arrivals_before, int* barriers_out, int* grid_out, int* status,
                            void* trace, int sm_count, void* stream) {
  if (world < 1 || world > DP_MAX || ngroups < 1 || ngroups > DP_MAX_GROUPS) return -3;
  if ((shard_lo % 4) || (shard_hi % 4) || (total % 4)) return -2;
  if (shard_lo < 0 || shard_hi < shard_lo || shard_hi > total) return -2;
  DpArgs a = {};
  a.rank = rank; a.world = world;
  for (int p = 0; p < world; ++p) {
    a.grad[p] = (float*)grad[p];
    a.master[p] = (float*)master[p];
    a.lp[p] = lp ? lp[p] : nullptr;
    a.flags[p] = (int*)flags[p];
  }
  a.m = (float*)m; a.v = (float*)v; a.local_sync = (int*)local_sync;
  a.shard_lo = shard_lo; a.shard_hi = shard_hi; a.total = total;
  a.ngroups = ngroups;
  for (int g = 0; g < ngroups; ++g) {
    DpGroup& G = a.group[g];
    G.lo = groups[4 * g]; G.hi = groups[4 * g + 1];
    G.local_below = groups[4 * g + 2]; G.master_from = groups[4 * g + 3];
    if ((G.lo % 4) || (G.hi % 4)) return -2;
    G.lr = hyper[6 * g]; G.beta1 = hyper[6 * g + 1]; G.beta2 = hyper[6 * g + 2];
    G.eps = hyper[6 * g + 3]; G.weight_decay = hyper[6 * g + 4]; G.adamw = hyper[6 * g + 5] != 0.f;
  }
  a.grad_scale = grad_scale; a.lp_dtype = lp_dtype;
  a.check_inf = check_inf; a.found_given = check_inf ? 0 : found_given;
  a.loss_scale = (const float*)loss_scale; a.found_inf = (float*)found_inf;
  a.applied_steps = (const int*)applied_steps; a.host_step = host_step;
  a.epoch = epoch; a.status = status; a.trace = (long long*)trace;
  // two 512-thread CTAs per SM: all CTAs are co-resident (the barriers rely on it; a CTA that
  // has to wait for an SM delays the barrier, within the wait limit)
  const int grid = 2 * (sm_count > 0 ? sm_count : 148);
  a.sync_base = arrivals_before;
  if (barriers_out) *barriers_out = 3;
  if (grid_out) *grid_out = grid;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (world) {
    case 1: dp_fused_kernel<1><<<grid, DP_THREADS, 0, st>>>(a); break;
    case 2: dp_fused_kernel<2><<<grid, DP_THREADS, 0, st>>>(a); break;
    case 3: dp_fused_kernel<3><<<grid, DP_THREADS, 0, st>>>(a); break;
    case 4: dp_fused_kernel<4><<<grid, DP_THREADS, 0, st>>>(a); break;
    case 5: dp_fused_kernel<5><<<grid, DP_THREADS, 0, st>>>(a); break;
    case 6: dp_fused_kernel<6><<<grid, DP_THREADS, 0, st>>>(a); break;
    case 7: dp_fused_kernel<7><<<grid, DP_THREADS, 0, st>>>(a); break;
    default: dp_fused_kernel<8><<<grid, DP_THREADS, 0, st>>>(a); break;
  }
  PF_CHECK_LAUNCH();
  return 0;
}

// ---- rows of a weight owned by other ranks, copied into the local copy (plain peer loads).
// Used when the first consumer of a freshly updated weight is not the fused all-gather GEMM.
namespace pf {
struct RowGatherArgs {
  const void* src[DP_MAX];     // every rank's full-size copy [rows, row_bytes]
  void* dst;                   // the local copy
  int row_end[DP_MAX];
  int world, rank, rows;
  long long row_bytes;         // multiple of 16
};
__global__ void __launch_bounds__(256)
row_gather_kernel(const RowGatherArgs a) {
  const long long vec_per_row = a.row_bytes / 16;
  const long long total = (long long)a.rows * vec_per_row;
  const int own0 = a.rank > 0 ? a.row_end[a.rank - 1] : 0, own1 = a.row_end[a.rank];
  const long long stride = (long long)gridDim.x * blockDim.x;
  constexpr int U = 4;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < total;
       i0 += stride * U) {
    uint4 buf[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      live[u] = false;
      if (i < total) {
        const int r = (int)(i / vec_per_row);
        if (r < own0 || r >= own1) {
          int owner = 0;
          while (owner < a.world - 1 && r >= a.row_end[owner]) ++owner;
          buf[u] = reinterpret_cast<const uint4*>(a.src[owner])[i];
          live[u] = true;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (live[u]) reinterpret_cast<uint4*>(a.dst)[i0 + u * stride] = buf[u];
  }
}
}  // namespace pf

PF_API int pf_gather_rows(void* dst, void* const* copies, const int* row_end, int world, int rank,
                          int rows, long long row_bytes, int sm_count, void* stream) {
  if (world < 1 || world > DP_MAX || row_bytes % 16) return -3;
  if (rows <= 0 || world == 1) return 0;
  RowGatherArgs a = {};
  for (int i = 0; i < DP_MAX; ++i) {
    a.src[i] = i < world ? copies[i] : nullptr;
    a.row_end[i] = i < world ? row_end[i] : rows;
  }
  a.dst = dst; a.world = world; a.rank = rank; a.rows = rows; a.row_bytes = row_bytes;
  const int grid = 4 * (sm_count > 0 ? sm_count : 148);
  row_gather_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  PF_CHECK_LAUNCH();
  return 0;
}

// ---- IPC plumbing for peer-visible buffers
PF_API int pf_ipc_get_handle(void* ptr, void* handle_out_64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out_64, &h, sizeof(h));
  return 0;
}
PF_API int pf_ipc_open(const void* handle_64, void** ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess);
  return (int)e;
}
PF_API int pf_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
PF_API int pf_get_base(void* ptr, void** base_out, long long* size_out) {
  // base address and size of the allocation that contains `ptr` (driver entry point looked up
  // at run time so the library does not link libcuda)
  typedef CUresult (*Fn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static Fn fn = nullptr;
  if (!fn) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return -100;
    fn = reinterpret_cast<Fn>(f);
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  CUresult r = fn(&base, &size, (CUdeviceptr)ptr);
  if (r != CUDA_SUCCESS) return -(1000 + (int)r);
  *base_out = (void*)base;
  *size_out = (long long)size;
  return 0;
}

// Reads 4 bytes at a (possibly peer-mapped) device address through the copy engine.  An
// unmapped address makes the copy return an error code; it does not fault the context.
PF_API int pf_peek_u32(const void* dev_ptr, unsigned int* out) {
  return (int)cudaMemcpy(out, dev_ptr, 4, cudaMemcpyDeviceToHost);
}
