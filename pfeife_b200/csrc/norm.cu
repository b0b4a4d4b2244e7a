// LayerNorm and RMSNorm, forward and backward, one CTA per row with the row held in registers
// (16-byte loads, two block reductions).  The forward can fuse the residual add of a
// pre-norm transformer block:  h = x + res ;  y = norm(h) * gamma (+ beta).
// The backward writes dx (optionally + the gradient that flows around the norm through the
// residual branch) and per-CTA partial sums of dgamma / dbeta into a scratch buffer that a
// second small kernel folds into the fp32 parameter gradients.
#include "no_alloc.h"
#include "common.cuh"
#include "api.h"

namespace pf {

constexpr int NORM_MAX_VEC = 4;   // 16-byte vectors per thread: N <= 256 * 4 * 8 = 8192 (16-bit)

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// rms != 0 -> RMSNorm (no mean subtraction, no beta)
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ res, const float* __restrict__ gamma,
                const float* __restrict__ beta, T* __restrict__ y, T* __restrict__ h_out,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int N, float eps,
                int rms) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int nvec = N / V;
  const T* xr = x + row * N;
  float vals[NORM_MAX_VEC][V];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      uint4 q = reinterpret_cast<const uint4*>(xr)[idx];
      const T* e = reinterpret_cast<const T*>(&q);
      if (res) {
        uint4 qr = reinterpret_cast<const uint4*>(res + row * N)[idx];
        const T* er = reinterpret_cast<const T*>(&qr);
        uint4 qh;
        T* eh = reinterpret_cast<T*>(&qh);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          // round the residual stream to its storage type first so fwd and bwd agree
          eh[j] = from_f32<T>(to_f32<T>(e[j]) + to_f32<T>(er[j]));
          vals[i][j] = to_f32<T>(eh[j]);
        }
        if (h_out) reinterpret_cast<uint4*>(h_out + row * N)[idx] = qh;
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) vals[i][j] = to_f32<T>(e[j]);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) s += vals[i][j];
    }
  }
  float mean = 0.f;
  if (!rms) mean = block_sum<THREADS>(s, red) / N;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float d = vals[i][j] - mean;
        sq += d * d;
      }
    }
  }
  const float var = block_sum<THREADS>(sq, red) / N;
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      uint4 q;
      T* e = reinterpret_cast<T*>(&q);
      const float4* g4 = reinterpret_cast<const float4*>(gamma + idx * V);
      float g[V], b[V];
#pragma unroll
      for (int j = 0; j < V / 4; ++j) {
        float4 t = __ldg(g4 + j);
        g[4 * j] = t.x; g[4 * j + 1] = t.y; g[4 * j + 2] = t.z; g[4 * j + 3] = t.w;
      }
      if (beta) {
        const float4* b4 = reinterpret_cast<const float4*>(beta + idx * V);
#pragma unroll
        for (int j = 0; j < V / 4; ++j) {
          float4 t = __ldg(b4 + j);
          b[4 * j] = t.x; b[4 * j + 1] = t.y; b[4 * j + 2] = t.z; b[4 * j + 3] = t.w;
        }
      }
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float o = (vals[i][j] - mean) * rstd * g[j];
        if (beta) o += b[j];
        e[j] = from_f32<T>(o);
      }
      reinterpret_cast<uint4*>(y + row * N)[idx] = q;
    }
  }
}

// Backward.  Grid = G persistent CTAs striding over rows; each thread keeps dgamma/dbeta
// partials for its own columns and writes them to scratch[blockIdx][2][N] at the end.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ h, const float* __restrict__ gamma,
                const float* __restrict__ mean, const float* __restrict__ rstd,
                const T* __restrict__ dres, T* __restrict__ dx, float* __restrict__ scratch,
                long long rows, int N, int rms) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float red[32];
  const int nvec = N / V;
  float dg[NORM_MAX_VEC][V], db[NORM_MAX_VEC][V], g[NORM_MAX_VEC][V];
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int idx = threadIdx.x + i * THREADS;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      dg[i][j] = 0.f; db[i][j] = 0.f;
      g[i][j] = (idx < nvec) ? gamma[idx * V + j] : 0.f;
    }
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mu = rms ? 0.f : mean[row];
    const float rs = rstd[row];
    float xh[NORM_MAX_VEC][V], dyv[NORM_MAX_VEC][V];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      if (idx < nvec) {
        uint4 qd = reinterpret_cast<const uint4*>(dy + row * N)[idx];
        uint4 qh = reinterpret_cast<const uint4*>(h + row * N)[idx];
        const T* ed = reinterpret_cast<const T*>(&qd);
        const T* eh = reinterpret_cast<const T*>(&qh);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float d = to_f32<T>(ed[j]);
          const float xhat = (to_f32<T>(eh[j]) - mu) * rs;
          xh[i][j] = xhat;
          dyv[i][j] = d * g[i][j];
          dg[i][j] += d * xhat;
          db[i][j] += d;
          s1 += dyv[i][j];
          s2 += dyv[i][j] * xhat;
        }
      }
    }
    float m1 = 0.f;
    if (!rms) m1 = block_sum<THREADS>(s1, red) / N;
    const float m2 = block_sum<THREADS>(s2, red) / N;
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      if (idx < nvec) {
        uint4 q;
        T* e = reinterpret_cast<T*>(&q);
        uint4 qr;
        const T* er = reinterpret_cast<const T*>(&qr);
        if (dres) qr = reinterpret_cast<const uint4*>(dres + row * N)[idx];
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float o = rs * (dyv[i][j] - m1 - xh[i][j] * m2);
          if (dres) o += to_f32<T>(er[j]);
          e[j] = from_f32<T>(o);
        }
        reinterpret_cast<uint4*>(dx + row * N)[idx] = q;
      }
    }
  }
  float* sg = scratch + (long long)blockIdx.x * 2 * N;
  float* sb = sg + N;
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        sg[idx * V + j] = dg[i][j];
        sb[idx * V + j] = db[i][j];
      }
    }
  }
}

// Forward for rows of up to 2048 16-bit elements: one warp per row, shuffle reductions only (no
// CTA barrier), 8 rows per CTA.  The row stays in registers in its packed 16-bit form and is
// expanded once per pass (sum, squared deviations, output): a third of the registers of an fp32
// copy, which lets enough CTAs share an SM to keep the loads of a whole wave in flight.
template <typename T, int NV>
__global__ void __launch_bounds__(256, 4)
norm_fwd_warp_kernel(const T* __restrict__ x, const T* __restrict__ res,
                     const float* __restrict__ gamma, const float* __restrict__ beta,
                     T* __restrict__ y, T* __restrict__ h_out, float* __restrict__ mean_out,
                     float* __restrict__ rstd_out, long long rows, int N, float eps, int rms) {
  constexpr int V = 8;
  const int nvec = N / V;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  uint4 q[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = lane + i * 32;
    if (idx < nvec) q[i] = reinterpret_cast<const uint4*>(x + row * N)[idx];
  }
  if (res) {      // h = x + residual, rounded to the storage type like the unfused sequence
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
        const uint4 qr = reinterpret_cast<const uint4*>(res + row * N)[idx];
        const T* er = reinterpret_cast<const T*>(&qr);
        T* e = reinterpret_cast<T*>(&q[i]);
#pragma unroll
        for (int j = 0; j < V; ++j) e[j] = from_f32<T>(to_f32<T>(e[j]) + to_f32<T>(er[j]));
        if (h_out) reinterpret_cast<uint4*>(h_out + row * N)[idx] = q[i];
      }
    }
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + i * 32 < nvec) {
      const T* e = reinterpret_cast<const T*>(&q[i]);
#pragma unroll
      for (int j = 0; j < V; ++j) s += to_f32<T>(e[j]);
    }
  }
  const float mean = rms ? 0.f : warp_sum(s) / N;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + i * 32 < nvec) {
      const T* e = reinterpret_cast<const T*>(&q[i]);
#pragma unroll
      for (int j = 0; j < V; ++j) { const float d = to_f32<T>(e[j]) - mean; sq = fmaf(d, d, sq); }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / N + eps);
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = lane + i * 32;
    if (idx < nvec) {
      const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + idx * V));
      const float4 g1 = __ldg(reinterpret_cast<const float4*>(gamma + idx * V) + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      float b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (beta) {
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta + idx * V));
        const float4 b1 = __ldg(reinterpret_cast<const float4*>(beta + idx * V) + 1);
        b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w;
        b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
      }
      const T* ei = reinterpret_cast<const T*>(&q[i]);
      uint4 o;
      T* e = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int j = 0; j < V; ++j)
        e[j] = from_f32<T>((to_f32<T>(ei[j]) - mean) * rstd * g[j] + b[j]);
      reinterpret_cast<uint4*>(y + row * N)[idx] = o;
    }
  }
}

// Backward, input gradient only: one warp per row, packed dy / h kept in registers, two
// shuffle reductions.  The parameter gradients come from norm_bwd_param_kernel.
template <typename T, int NV>
__global__ void __launch_bounds__(256)
norm_bwd_dx_kernel(const T* __restrict__ dy, const T* __restrict__ h,
                   const float* __restrict__ gamma, const float* __restrict__ mean,
                   const float* __restrict__ rstd, const T* __restrict__ dres,
                   T* __restrict__ dx, long long rows, int N, int rms) {
  constexpr int V = 8;
  const int nvec = N / V;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float mu = rms ? 0.f : mean[row];
  const float rs = rstd[row];
  uint4 qd[NV], qh[NV];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = lane + i * 32;
    if (idx < nvec) {
      qd[i] = reinterpret_cast<const uint4*>(dy + row * N)[idx];
      qh[i] = reinterpret_cast<const uint4*>(h + row * N)[idx];
      const T* ed = reinterpret_cast<const T*>(&qd[i]);
      const T* eh = reinterpret_cast<const T*>(&qh[i]);
      const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + idx * V));
      const float4 g1 = __ldg(reinterpret_cast<const float4*>(gamma + idx * V) + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float dyg = to_f32<T>(ed[j]) * g[j];
        s1 += dyg;
        s2 += dyg * (to_f32<T>(eh[j]) - mu) * rs;
      }
    }
  }
  const float m1 = rms ? 0.f : warp_sum(s1) / N;
  const float m2 = warp_sum(s2) / N;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = lane + i * 32;
    if (idx < nvec) {
      const T* ed = reinterpret_cast<const T*>(&qd[i]);
      const T* eh = reinterpret_cast<const T*>(&qh[i]);
      const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + idx * V));
      const float4 g1 = __ldg(reinterpret_cast<const float4*>(gamma + idx * V) + 1);
      const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      uint4 qr;
      if (dres) qr = reinterpret_cast<const uint4*>(dres + row * N)[idx];
      const T* er = reinterpret_cast<const T*>(&qr);
      uint4 q;
      T* e = reinterpret_cast<T*>(&q);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float xhat = (to_f32<T>(eh[j]) - mu) * rs;
        float o = rs * (to_f32<T>(ed[j]) * g[j] - m1 - xhat * m2);
        if (dres) o += to_f32<T>(er[j]);
        e[j] = from_f32<T>(o);
      }
      reinterpret_cast<uint4*>(dx + row * N)[idx] = q;
    }
  }
}

// dgamma[c] += sum_r dy[r,c] * xhat[r,c] ; dbeta[c] += sum_r dy[r,c].  Each CTA owns 256
// columns (lane = 8 consecutive columns, 16-byte loads) and a slab of rows split over its 8
// warps; warps are combined through shared memory and the CTA writes its partial sums to the
// scratch buffer, which norm_bwd_finish_kernel folds (deterministic, nothing to zero).
template <typename T>
__global__ void __launch_bounds__(256)
norm_bwd_param_kernel(const T* __restrict__ dy, const T* __restrict__ h,
                      const float* __restrict__ mean, const float* __restrict__ rstd,
                      float* __restrict__ scratch, float* __restrict__ acc_gamma,
                      float* __restrict__ acc_beta, long long rows, int N, int rows_per_cta,
                      int rms) {
  __shared__ float red[2][8][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 256 + lane * 8;
  const long long r0 = (long long)blockIdx.y * rows_per_cta;
  const long long r1 = min(rows, r0 + rows_per_cta);
  float ag[8] = {0, 0, 0, 0, 0, 0, 0, 0}, ab[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c0 < N) {
    for (long long r = r0 + warp; r < r1; r += 8) {
      const float mu = rms ? 0.f : mean[r];
      const float rs = rstd[r];
      const uint4 qd = *reinterpret_cast<const uint4*>(dy + r * N + c0);
      const uint4 qh = *reinterpret_cast<const uint4*>(h + r * N + c0);
      const T* ed = reinterpret_cast<const T*>(&qd);
      const T* eh = reinterpret_cast<const T*>(&qh);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = to_f32<T>(ed[j]);
        ag[j] += d * (to_f32<T>(eh[j]) - mu) * rs;
        ab[j] += d;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    red[0][warp][lane * 8 + j] = ag[j];
    red[1][warp][lane * 8 + j] = ab[j];
  }
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < N) {
    float g = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { g += red[0][w][threadIdx.x]; b += red[1][w][threadIdx.x]; }
    if (acc_gamma) {
      // accumulating into existing gradients (the framework's gradient bucket): add this row
      // slab's sums directly, no folding pass
      atomicAdd(acc_gamma + c, g);
      if (acc_beta) atomicAdd(acc_beta + c, b);
    } else {
      // partial sums of this row slab: scratch[slab][0][c] (dgamma), scratch[slab][1][c] (dbeta)
      scratch[((long long)blockIdx.y * 2) * N + c] = g;
      scratch[((long long)blockIdx.y * 2 + 1) * N + c] = b;
    }
  }
}

// Backward for rows of up to 2048 16-bit elements: one WARP per row (no CTA-wide barrier on the
// row path), 8 warps per CTA, rows strided over a persistent grid.  Each lane keeps the packed
// dy / h vectors of its row slice in registers, expands them twice (reduction pass, output
// pass) and carries dgamma / dbeta partials for its columns across rows.  At the end the 8
// warps of a CTA fold their partials through shared memory into scratch[blockIdx][2][N].
template <typename T, int NV>
__global__ void __launch_bounds__(256)
norm_bwd_warp_kernel(const T* __restrict__ dy, const T* __restrict__ h,
                     const float* __restrict__ gamma, const float* __restrict__ mean,
                     const float* __restrict__ rstd, const T* __restrict__ dres,
                     T* __restrict__ dx, float* __restrict__ scratch, long long rows, int N,
                     int rms) {
  constexpr int V = 16 / sizeof(T);
  extern __shared__ float sacc[];          // [2][N]
  const int nvec = N / V;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 2 * N; i += 256) sacc[i] = 0.f;
  __syncthreads();
  float dg[NV][V], db[NV][V];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < V; ++j) { dg[i][j] = 0.f; db[i][j] = 0.f; }
  const float inv_n = 1.f / N;
  for (long long row = (long long)blockIdx.x * 8 + warp; row < rows;
       row += (long long)gridDim.x * 8) {
    const float mu = rms ? 0.f : mean[row];
    const float rs = rstd[row];
    uint4 qd[NV], qh[NV];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
        qd[i] = reinterpret_cast<const uint4*>(dy + row * N)[idx];
        qh[i] = reinterpret_cast<const uint4*>(h + row * N)[idx];
        const T* ed = reinterpret_cast<const T*>(&qd[i]);
        const T* eh = reinterpret_cast<const T*>(&qh[i]);
        const float4* g4 = reinterpret_cast<const float4*>(gamma + idx * V);
#pragma unroll
        for (int j4 = 0; j4 < V / 4; ++j4) {
          const float4 g = __ldg(g4 + j4);
          const float gg[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = j4 * 4 + u;
            const float d = to_f32<T>(ed[j]);
            const float xhat = (to_f32<T>(eh[j]) - mu) * rs;
            const float dyg = d * gg[u];
            s1 += dyg;
            s2 += dyg * xhat;
            dg[i][j] += d * xhat;
            db[i][j] += d;
          }
        }
      }
    }
    const float m1 = rms ? 0.f : warp_sum(s1) * inv_n;
    const float m2 = warp_sum(s2) * inv_n;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
        const T* ed = reinterpret_cast<const T*>(&qd[i]);
        const T* eh = reinterpret_cast<const T*>(&qh[i]);
        uint4 qr;
        if (dres) qr = reinterpret_cast<const uint4*>(dres + row * N)[idx];
        const T* er = reinterpret_cast<const T*>(&qr);
        uint4 q;
        T* e = reinterpret_cast<T*>(&q);
        const float4* g4 = reinterpret_cast<const float4*>(gamma + idx * V);
#pragma unroll
        for (int j4 = 0; j4 < V / 4; ++j4) {
          const float4 g = __ldg(g4 + j4);
          const float gg[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = j4 * 4 + u;
            const float xhat = (to_f32<T>(eh[j]) - mu) * rs;
            float o = rs * (to_f32<T>(ed[j]) * gg[u] - m1 - xhat * m2);
            if (dres) o += to_f32<T>(er[j]);
            e[j] = from_f32<T>(o);
          }
        }
        reinterpret_cast<uint4*>(dx + row * N)[idx] = q;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int idx = lane + i * 32;
    if (idx < nvec) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        atomicAdd(&sacc[idx * V + j], dg[i][j]);
        atomicAdd(&sacc[N + idx * V + j], db[i][j]);
      }
    }
  }
  __syncthreads();
  float* out = scratch + (long long)blockIdx.x * 2 * N;
  for (int i = threadIdx.x; i < 2 * N; i += 256) out[i] = sacc[i];
}

// dgamma[c] (+)= sum_g scratch[g][0][c] ; dbeta likewise
__global__ void __launch_bounds__(256)
norm_bwd_finish_kernel(const float* __restrict__ scratch, float* __restrict__ dgamma,
                       float* __restrict__ dbeta, int G, int N, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float a = 0.f, b = 0.f;
  for (int g = 0; g < G; ++g) {
    a += scratch[(long long)g * 2 * N + c];
    b += scratch[(long long)g * 2 * N + N + c];
  }
  dgamma[c] = accumulate ? dgamma[c] + a : a;
  if (dbeta) dbeta[c] = accumulate ? dbeta[c] + b : b;
}

template <typename T>
static int norm_fwd_launch(const void* x, const void* res, const float* gamma, const float* beta,
                           void* y, void* h_out, float* mean, float* rstd, long long rows, int N,
                           float eps, int rms, cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  if (N % V) return -2;
  const int nvec = N / V;
  if (sizeof(T) == 2 && nvec <= 32 * 8) {
    const unsigned grid = (unsigned)((rows + 7) / 8);
#define PF_NORM_FWD_WARP(NV)                                                                  \
    norm_fwd_warp_kernel<T, NV><<<grid, 256, 0, st>>>((const T*)x, (const T*)res, gamma, beta, \
        (T*)y, (T*)h_out, mean, rstd, rows, N, eps, rms)
    if (nvec <= 32 * 2) PF_NORM_FWD_WARP(2);
    else if (nvec <= 32 * 4) PF_NORM_FWD_WARP(4);
    else if (nvec <= 32 * 6) PF_NORM_FWD_WARP(6);
    else PF_NORM_FWD_WARP(8);
#undef PF_NORM_FWD_WARP
    return 0;
  }
  if (nvec <= 128 * NORM_MAX_VEC)
    norm_fwd_kernel<T, 128><<<(unsigned)rows, 128, 0, st>>>((const T*)x, (const T*)res, gamma,
        beta, (T*)y, (T*)h_out, mean, rstd, N, eps, rms);
  else if (nvec <= 256 * NORM_MAX_VEC)
    norm_fwd_kernel<T, 256><<<(unsigned)rows, 256, 0, st>>>((const T*)x, (const T*)res, gamma,
        beta, (T*)y, (T*)h_out, mean, rstd, N, eps, rms);
  else if (nvec <= 1024 * NORM_MAX_VEC)
    norm_fwd_kernel<T, 1024><<<(unsigned)rows, 1024, 0, st>>>((const T*)x, (const T*)res, gamma,
        beta, (T*)y, (T*)h_out, mean, rstd, N, eps, rms);
  else
    return -3;
  return 0;
}

template <typename T>
static int norm_bwd_launch(const void* dy, const void* h, const float* gamma, const float* mean,
                           const float* rstd, const void* dres, void* dx, float* scratch, int& G,
                           long long rows, int N, int rms, cudaStream_t st,
                           float* acc_gamma = nullptr, float* acc_beta = nullptr) {
  constexpr int V = 16 / sizeof(T);
  if (N % V) return -2;
  const int nvec = N / V;
  if (sizeof(T) == 2 && nvec <= 32 * 16) {
    // input gradient: warp per row (rows of up to 4096 16-bit elements: Llama's hidden size);
    // parameter gradients: column reduction over row slabs
    const unsigned grid = (unsigned)((rows + 7) / 8);
#define PF_NORM_BWD_DX(NV)                                                                   \
    norm_bwd_dx_kernel<T, NV><<<grid, 256, 0, st>>>((const T*)dy, (const T*)h, gamma, mean,  \
        rstd, (const T*)dres, (T*)dx, rows, N, rms)
    if (nvec <= 32 * 2) PF_NORM_BWD_DX(2);
    else if (nvec <= 32 * 4) PF_NORM_BWD_DX(4);
    else if (nvec <= 32 * 6) PF_NORM_BWD_DX(6);
    else if (nvec <= 32 * 8) PF_NORM_BWD_DX(8);
    else if (nvec <= 32 * 12) PF_NORM_BWD_DX(12);
    else PF_NORM_BWD_DX(16);
#undef PF_NORM_BWD_DX
    // enough row slabs to fill the GPU once with (column blocks x slabs) CTAs, few enough
    // that folding them (norm_bwd_finish_kernel) stays negligible
    const int col_blocks = (N + 255) / 256;
    int slabs = (2 * 148 + col_blocks - 1) / col_blocks;
    if (slabs > (int)((rows + 31) / 32)) slabs = (int)((rows + 31) / 32);
    if (slabs > G) slabs = G;
    if (slabs < 1) slabs = 1;
    const int rows_per = (int)((rows + slabs - 1) / slabs);
    slabs = (int)((rows + rows_per - 1) / rows_per);
    norm_bwd_param_kernel<T><<<dim3((N + 255) / 256, slabs), 256, 0, st>>>(
        (const T*)dy, (const T*)h, mean, rstd, scratch, acc_gamma, acc_beta, rows, N, rows_per,
        rms);
    G = acc_gamma ? 0 : slabs;      // 0: the sums are already where they belong
    return 0;
  }
  if (nvec <= 128 * NORM_MAX_VEC)
    norm_bwd_kernel<T, 128><<<G, 128, 0, st>>>((const T*)dy, (const T*)h, gamma, mean, rstd,
        (const T*)dres, (T*)dx, scratch, rows, N, rms);
  else if (nvec <= 256 * NORM_MAX_VEC)
    norm_bwd_kernel<T, 256><<<G, 256, 0, st>>>((const T*)dy, (const T*)h, gamma, mean, rstd,
        (const T*)dres, (T*)dx, scratch, rows, N, rms);
  else if (nvec <= 1024 * NORM_MAX_VEC)
    norm_bwd_kernel<T, 1024><<<G, 1024, 0, st>>>((const T*)dy, (const T*)h, gamma, mean, rstd,
        (const T*)dres, (T*)dx, scratch, rows, N, rms);
  else
    return -3;
  return 0;
}

}  // namespace pf

using namespace pf;

PF_API int pf_norm_fwd(const void* x, const void* res, const void* gamma, const void* beta,
                       void* y, void* h_out, void* mean, void* rstd, long long rows, int N,
                       float eps, int rms, int dtype, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int r = -1;
  switch (dtype) {
    case PF_F32: r = norm_fwd_launch<float>(x, res, (const float*)gamma, (const float*)beta, y, h_out, (float*)mean, (float*)rstd, rows, N, eps, rms, st); break;
    case PF_F16: r = norm_fwd_launch<__half>(x, res, (const float*)gamma, (const float*)beta, y, h_out, (float*)mean, (float*)rstd, rows, N, eps, rms, st); break;
    case PF_BF16: r = norm_fwd_launch<__nv_bfloat16>(x, res, (const float*)gamma, (const float*)beta, y, h_out, (float*)mean, (float*)rstd, rows, N, eps, rms, st); break;
  }
  if (r) return r;
  PF_CHECK_LAUNCH();
  return 0;
}

// Number of CTAs (= rows of the scratch buffer) the backward uses for `rows` rows.
PF_API int pf_norm_bwd_ctas(long long rows, int sm_count) {
  long long g = (long long)(sm_count > 0 ? sm_count : 148) * 2;
  if (g > (rows + 7) / 8) g = (rows + 7) / 8;
  if (g < 1) g = 1;
  return (int)g;
}

// scratch: fp32 [pf_norm_bwd_ctas(rows)][2][N], contents on entry irrelevant.
PF_API int pf_norm_bwd(const void* dy, const void* h, const void* gamma, const void* mean,
                       const void* rstd, const void* dres, void* dx, void* dgamma, void* dbeta,
                       void* scratch, long long rows, int N, int rms, int accumulate, int dtype,
                       int sm_count, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int G = pf_norm_bwd_ctas(rows, sm_count);   // rows of scratch; the launch may use fewer
  // when the sums are added to existing gradients the row slabs add them directly (G comes
  // back 0) instead of leaving partial sums for the folding kernel
  float* ag = accumulate ? (float*)dgamma : nullptr;
  float* ab = accumulate ? (float*)dbeta : nullptr;
  int r = -1;
  switch (dtype) {
    case PF_F32: r = norm_bwd_launch<float>(dy, h, (const float*)gamma, (const float*)mean, (const float*)rstd, dres, dx, (float*)scratch, G, rows, N, rms, st, ag, ab); break;
    case PF_F16: r = norm_bwd_launch<__half>(dy, h, (const float*)gamma, (const float*)mean, (const float*)rstd, dres, dx, (float*)scratch, G, rows, N, rms, st, ag, ab); break;
    case PF_BF16: r = norm_bwd_launch<__nv_bfloat16>(dy, h, (const float*)gamma, (const float*)mean, (const float*)rstd, dres, dx, (float*)scratch, G, rows, N, rms, st, ag, ab); break;
  }
  if (r) return r;
  PF_CHECK_LAUNCH();
  if (G > 0) {
    norm_bwd_finish_kernel<<<(N + 255) / 256, 256, 0, st>>>((const float*)scratch, (float*)dgamma,
                                                            (float*)dbeta, G, N, accumulate);
    PF_CHECK_LAUNCH();
  }
  return 0;
}

// ------------------------------------------------------------------ allocation-free variant

// Partial dgamma / dbeta sums of pf_norm_bwd_static.  One copy per device that loads the
// library; shared by every call on that device.
static __device__ __align__(256) float g_norm_static_scratch[PF_NORM_STATIC_SCRATCH_FLOATS];

// In host code `g_norm_static_scratch` is only a handle for the runtime's symbol table, not
// a device address; the address is queried once per device, with that device current.
static float* norm_static_scratch_ptr(int* err) {
  static float* ptrs[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) { *err = e != cudaSuccess ? (int)e : -3; return nullptr; }
  if (!ptrs[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_norm_static_scratch);
    if (e != cudaSuccess) { *err = (int)e; return nullptr; }
    ptrs[dev] = static_cast<float*>(p);
  }
  *err = 0;
  return ptrs[dev];
}

PF_API int pf_norm_bwd_static(const void* dy, const void* h, const void* gamma, const void* mean,
                              const void* rstd, const void* dres, void* dx, void* dgamma,
                              void* dbeta, long long rows, int N, int rms, int accumulate,
                              int dtype, int sm_count, void* stream) {
  if (rows <= 0) return 0;
  const long long need = (long long)pf_norm_bwd_ctas(rows, sm_count) * 2 * N;
  if (need > PF_NORM_STATIC_SCRATCH_FLOATS) return -3;   // beyond the built-in scratch
  int err = 0;
  float* scratch = norm_static_scratch_ptr(&err);
  if (!scratch) return err;
  return pf_norm_bwd(dy, h, gamma, mean, rstd, dres, dx, dgamma, dbeta, scratch, rows, N, rms,
                     accumulate, dtype, sm_count, stream);
}
