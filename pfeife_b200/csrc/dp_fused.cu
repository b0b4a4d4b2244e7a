// Fused data-parallel step over NVLink peer memory: gradient reduce-scatter + unscale +
// non-finite agreement + partitioned AdamW + all-gather of the updated weights, in ONE kernel
// per rank (one process per GPU; every rank launches the same kernel on its own stream).
//
// Every rank owns a contiguous shard of the flat parameter space.  Its kernel
//   1. waits until every rank has finished its backward (flag barrier over peer memory),
//   2. reads its shard of the fp32 gradient bucket from EVERY rank with plain P2P vector loads,
//      sums, stores the sum into its own bucket and zeroes the peers' copies (ready for the
//      next step's accumulation), noting whether anything was non-finite,
//   3. publishes its non-finite flag to all ranks and barriers, so that all ranks take the same
//      skip decision (dynamic loss scaling),
//   4. applies AdamW on the shard with moments that exist only on the owner (ZeRO-1 memory),
//      and writes the new fp32 master weights and their 16-bit shadow into EVERY rank's
//      buffers with P2P vector stores,
//   5. barriers again so nobody starts the next forward on half-written weights.
// No NCCL call, no TMA and no multicast load is involved; all remote traffic is ld/st.global on
// IPC-mapped peer pointers.  Barriers are epoch counters written with st.release.sys and
// polled with ld.acquire.sys; every poll is bounded and reports PF_ERR_TIMEOUT_PEER_FLAG
// instead of spinning forever when a peer is gone.
#include <cstring>
#include "common.cuh"
#include "api.h"

namespace pf {

constexpr int DP_MAX = 8;
// Ranks reach the first barrier of a step with the skew of a whole training step between
// them (first-step compilation, graph capture), so that wait is allowed ~20 s; the later
// barriers only cover the kernel's own phases.
constexpr long long DP_ENTRY_WAIT = 20 * PF_WAIT_CYCLES;
constexpr int DP_THREADS = 512;

struct DpArgs {
  int rank, world;
  float* grad[DP_MAX];
  float* master[DP_MAX];
  void* lp[DP_MAX];            // null when there is no 16-bit shadow
  int* flags[DP_MAX];          // per rank: int[DP_MAX] barrier slots + int[DP_MAX] found slots
  float* m;                    // local moments, indexed from shard_lo
  float* v;
  int* local_sync;             // local: [0] arrival counter, [1] release word
  long long shard_lo, shard_hi;
  long long local_below;       // 16-bit weights at flat indices below this are written locally
                               // only: their first consumer gathers the rows other ranks own
                               // (fused all-gather GEMM); fp32 masters always go to every rank
  long long zero_lo, zero_hi;  // range of the local gradient bucket this call clears
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale;
  int adamw, lp_dtype, check_inf;
  const float* loss_scale;     // local device scalar (identical on every rank) or null
  float* found_inf;            // local: set to 1 when the step was skipped
  int epoch;                   // barrier epoch base of this call (strictly increasing)
  int sync_base;               // arrivals expected before this call
  int* status;
};

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

// All CTAs of this GPU and all ranks meet here.  `k` = ordinal of the barrier within the call.
__device__ void job_barrier(const DpArgs& a, int k) {
  __threadfence_system();
  __syncthreads();
  const int epoch = a.epoch + k;
  if (threadIdx.x == 0) {
    const int target = a.sync_base + (k + 1) * gridDim.x;
    atomicAdd(&a.local_sync[0], 1);
    if (blockIdx.x == 0) {
      long long t0 = clock64();
      bool ok = true;
      while (ld_acquire_gpu(&a.local_sync[0]) < target) {
        if (clock64() - t0 > PF_WAIT_CYCLES) { report(a.status, PF_ERR_TIMEOUT_PEER_FLAG); ok = false; break; }
      }
      __threadfence_system();
      for (int p = 0; p < a.world; ++p) st_release_sys(&a.flags[p][a.rank], epoch);
      const long long limit = (k == 0) ? DP_ENTRY_WAIT : PF_WAIT_CYCLES;
      for (int r = 0; r < a.world && ok; ++r) {
        t0 = clock64();
        while (ld_acquire_sys(&a.flags[a.rank][r]) < epoch) {
          if (clock64() - t0 > limit) { report(a.status, PF_ERR_TIMEOUT_PEER_FLAG); ok = false; break; }
        }
      }
      __threadfence_system();
      atomicExch(&a.local_sync[1], epoch);
    } else {
      long long t0 = clock64();
      while (ld_acquire_gpu(&a.local_sync[1]) < epoch) {
        if (clock64() - t0 > ((k == 0) ? DP_ENTRY_WAIT : PF_WAIT_CYCLES) * (a.world + 1)) { report(a.status, PF_ERR_TIMEOUT_PEER_FLAG); break; }
      }
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(DP_THREADS, 2)
dp_fused_kernel(const DpArgs a) {
  const long long lo = a.shard_lo, hi = a.shard_hi;
  const long long nvec = (hi - lo) / 4;        // shards are multiples of 4 elements
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;

  job_barrier(a, 0);                            // every rank's gradients are complete

  // ---- reduce-scatter into the local bucket, zero the peers' copies.  Four 16-byte vectors
  //      per thread and peer are requested before any is consumed, so enough bytes are in
  //      flight to cover the NVLink latency.
  bool bad = false;
  constexpr int U = 4;
  for (long long i0 = tid; i0 < nvec; i0 += stride * U) {
    float4 s[U];
#pragma unroll
    for (int u = 0; u < U; ++u) s[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < a.world; ++p) {
      float4 g[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        g[u] = i < nvec ? *reinterpret_cast<const float4*>(a.grad[p] + lo + i * 4)
                        : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        s[u].x += g[u].x; s[u].y += g[u].y; s[u].z += g[u].z; s[u].w += g[u].w;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nvec) {
        *reinterpret_cast<float4*>(a.grad[a.rank] + lo + i * 4) = s[u];
        if (a.check_inf)
          bad |= !(isfinite(s[u].x) && isfinite(s[u].y) && isfinite(s[u].z) && isfinite(s[u].w));
      }
    }
  }
  if (a.check_inf) {
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0)
      for (int p = 0; p < a.world; ++p) st_release_sys(&a.flags[p][DP_MAX + a.rank], a.epoch);
  }

  job_barrier(a, 1);                            // everybody's non-finite flag is published

  // ---- every rank has read what it needed of this bucket: clear the part of it that other
  //      ranks own (local stores; the own shard is cleared by the update loop below)
  {
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const long long n_before = (lo - a.zero_lo) / 4, n_after = (a.zero_hi - hi) / 4;
    for (long long i = tid; i < n_before; i += stride)
      *reinterpret_cast<float4*>(a.grad[a.rank] + a.zero_lo + i * 4) = z4;
    for (long long i = tid; i < n_after; i += stride)
      *reinterpret_cast<float4*>(a.grad[a.rank] + hi + i * 4) = z4;
  }

  bool skip = false;
  if (a.check_inf) {
    for (int r = 0; r < a.world; ++r)
      skip |= ld_acquire_sys(&a.flags[a.rank][DP_MAX + r]) == a.epoch;
    if (tid == 0) *a.found_inf = skip ? 1.f : 0.f;
  }
  float gs = a.grad_scale;
  if (a.loss_scale) gs /= *a.loss_scale;
  const float inv_bc1 = 1.f / a.bc1;
  const float inv_sqrt_bc2 = rsqrtf(a.bc2);

  // ---- partitioned AdamW, all-gather of master weights and 16-bit shadow by P2P stores
  for (long long i = tid; i < nvec; i += stride) {
    const long long e = lo + i * 4;
    float4 g4 = *reinterpret_cast<const float4*>(a.grad[a.rank] + e);
    *reinterpret_cast<float4*>(a.grad[a.rank] + e) = make_float4(0.f, 0.f, 0.f, 0.f);
    if (skip) continue;
    float4 w4 = *reinterpret_cast<const float4*>(a.master[a.rank] + e);
    float4 m4 = *reinterpret_cast<const float4*>(a.m + i * 4);
    float4 v4 = *reinterpret_cast<const float4*>(a.v + i * 4);
    float g[4] = {g4.x, g4.y, g4.z, g4.w}, w[4] = {w4.x, w4.y, w4.z, w4.w};
    float m[4] = {m4.x, m4.y, m4.z, m4.w}, v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gr = g[j] * gs;
      if (a.adamw) w[j] *= (1.f - a.lr * a.weight_decay);
      else gr += a.weight_decay * w[j];
      m[j] = a.beta1 * m[j] + (1.f - a.beta1) * gr;
      v[j] = a.beta2 * v[j] + (1.f - a.beta2) * gr * gr;
      w[j] -= a.lr * (m[j] * inv_bc1) / (sqrtf(v[j]) * inv_sqrt_bc2 + a.eps);
    }
    *reinterpret_cast<float4*>(a.m + i * 4) = make_float4(m[0], m[1], m[2], m[3]);
    *reinterpret_cast<float4*>(a.v + i * 4) = make_float4(v[0], v[1], v[2], v[3]);
    const float4 nw = make_float4(w[0], w[1], w[2], w[3]);
    uint2 q = make_uint2(0, 0);
    if (a.lp[a.rank]) {
      if (a.lp_dtype == PF_BF16) {
        __nv_bfloat162 x = __floats2bfloat162_rn(w[0], w[1]), y = __floats2bfloat162_rn(w[2], w[3]);
        q = make_uint2(*reinterpret_cast<uint32_t*>(&x), *reinterpret_cast<uint32_t*>(&y));
      } else {
        __half2 x = __floats2half2_rn(w[0], w[1]), y = __floats2half2_rn(w[2], w[3]);
        q = make_uint2(*reinterpret_cast<uint32_t*>(&x), *reinterpret_cast<uint32_t*>(&y));
      }
    }
    const bool push_lp = e >= a.local_below;
    for (int p = 0; p < a.world; ++p) {
      *reinterpret_cast<float4*>(a.master[p] + e) = nw;
      if (a.lp[p] && (push_lp || p == a.rank))
        *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(a.lp[p]) + e) = q;
    }
  }

  job_barrier(a, 2);                            // all weights have landed everywhere
}

}  // namespace pf

using namespace pf;

// Pointer tables are arrays of `world` device pointers (entry `rank` is the local buffer).
// [shard_lo, shard_hi) is the part of this call's range [zero_lo, zero_hi) that this rank owns:
// it reduces and updates its shard and clears the whole range of its own gradient bucket.
// `epoch` must grow by at least 3 per call and be identical on every rank; `sync_base` is
// (number of earlier calls) * 3 * grid.  Returns the grid size used through *grid_out.
PF_API int pf_dp_fused_step(int rank, int world, void* const* grad, void* const* master,
                            void* const* lp, void* const* flags, void* m, void* v,
                            void* local_sync, long long shard_lo, long long shard_hi,
                            long long local_below, long long zero_lo, long long zero_hi,
                            float lr,
                            float beta1, float beta2, float eps, float weight_decay, int step,
                            float grad_scale, int adamw, int lp_dtype, int check_inf,
                            const void* loss_scale, void* found_inf, int epoch, int calls_before,
                            int* status, int sm_count, void* stream) {
  if (world < 1 || world > DP_MAX) return -3;
  if ((shard_lo % 4) || (shard_hi % 4)) return -2;
  DpArgs a = {};
  a.rank = rank; a.world = world;
  for (int p = 0; p < world; ++p) {
    a.grad[p] = (float*)grad[p];
    a.master[p] = (float*)master[p];
    a.lp[p] = lp ? lp[p] : nullptr;
    a.flags[p] = (int*)flags[p];
  }
  a.m = (float*)m; a.v = (float*)v; a.local_sync = (int*)local_sync;
  a.shard_lo = shard_lo; a.shard_hi = shard_hi;
  if (zero_lo > shard_lo || zero_hi < shard_hi || (zero_lo % 4) || (zero_hi % 4)) return -2;
  a.local_below = local_below;
  a.zero_lo = zero_lo; a.zero_hi = zero_hi;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.grad_scale = grad_scale; a.adamw = adamw; a.lp_dtype = lp_dtype; a.check_inf = check_inf;
  a.loss_scale = (const float*)loss_scale; a.found_inf = (float*)found_inf;
  a.epoch = epoch; a.status = status;
  // two 512-thread CTAs per SM: all CTAs are co-resident (the barriers rely on it)
  const int grid = 2 * (sm_count > 0 ? sm_count : 148);
  a.sync_base = calls_before * 3 * grid;
  dp_fused_kernel<<<grid, DP_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
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
