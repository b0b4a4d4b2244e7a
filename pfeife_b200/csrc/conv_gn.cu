// UNet support kernels, channels-last (NHWC) throughout:
//   * im2col / col2im for KxK convolutions: the convolution itself runs on the tcgen05 GEMM
//     (forward: cols . W^T ; dgrad: dY . W -> col2im ; wgrad: dY^T . cols accumulated in fp32).
//     1x1 convolutions skip these kernels entirely (they are plain GEMMs on the NHWC tensor).
//   * GroupNorm with optional fused SiLU, forward and backward.
//   * nearest-neighbour 2x upsampling and its backward.
#include "common.cuh"
#include "api.h"

namespace pf {

// cols[(b, ho, wo), (r, s, c)] = x[b, ho*stride - pad + r, wo*stride - pad + s, c]  (0 outside)
// One thread moves 8 channels (16 bytes).
template <typename T>
__global__ void __launch_bounds__(256)
im2col_kernel(const T* __restrict__ x, T* __restrict__ cols, int B, int H, int W, int C, int KH,
              int KW, int Ho, int Wo, int stride, int pad, long long ldc) {
  const int cv = C / 8;
  const long long total = (long long)B * Ho * Wo * KH * KW * cv;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
    const int c8 = (int)(i % cv);
    long long t = i / cv;
    const int s = (int)(t % KW); t /= KW;
    const int r = (int)(t % KH); t /= KH;
    const int wo = (int)(t % Wo); t /= Wo;
    const int ho = (int)(t % Ho);
    const int b = (int)(t / Ho);
    const int hi = ho * stride - pad + r, wi = wo * stride - pad + s;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (hi >= 0 && hi < H && wi >= 0 && wi < W)
      v = reinterpret_cast<const uint4*>(x + (((long long)b * H + hi) * W + wi) * C)[c8];
    const long long row = ((long long)b * Ho + ho) * Wo + wo;
    reinterpret_cast<uint4*>(cols + row * ldc + ((long long)r * KW + s) * C)[c8] = v;
  }
}

// dx[b, hi, wi, c] = sum over (r, s) of dcols[(b, ho, wo), (r, s, c)] with hi = ho*stride-pad+r
// Gather form (no atomics): each thread owns 8 channels of one input pixel.
template <typename T>
__global__ void __launch_bounds__(256)
col2im_kernel(const T* __restrict__ dcols, T* __restrict__ dx, int B, int H, int W, int C, int KH,
              int KW, int Ho, int Wo, int stride, int pad, long long ldc) {
  const int cv = C / 8;
  const long long total = (long long)B * H * W * cv;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
    const int c8 = (int)(i % cv);
    long long t = i / cv;
    const int wi = (int)(t % W); t /= W;
    const int hi = (int)(t % H);
    const int b = (int)(t / H);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < KH; ++r) {
      const int hn = hi + pad - r;
      if (hn < 0 || hn % stride) continue;
      const int ho = hn / stride;
      if (ho >= Ho) continue;
      for (int s = 0; s < KW; ++s) {
        const int wn = wi + pad - s;
        if (wn < 0 || wn % stride) continue;
        const int wo = wn / stride;
        if (wo >= Wo) continue;
        const long long row = ((long long)b * Ho + ho) * Wo + wo;
        uint4 q = reinterpret_cast<const uint4*>(dcols + row * ldc + ((long long)r * KW + s) * C)[c8];
        const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += to_f32<T>(e[j]);
      }
    }
    uint4 o;
    T* e = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(acc[j]);
    reinterpret_cast<uint4*>(dx + (((long long)b * H + hi) * W + wi) * C)[c8] = o;
  }
}

// ------------------------------------------------------------------------------ GroupNorm
// NHWC, C a multiple of 8.  All four passes read 16 bytes (8 channels) per thread and request.
//
// The statistics passes give every thread one fixed 8-channel vector and a stripe of pixels:
// the CTA is (C/8) columns x R rows of threads, a grid of (slabs, B) CTAs splits the pixels of
// each image, per-channel partial sums meet in shared memory, and one thread per group folds
// its channels and adds the result to the global sums (zeroed by the host function).

// threads per CTA for the statistics passes: a whole number of rows of C/8 threads
static inline int gn_rows(int C) { const int ncv = C / 8; return ncv >= 256 ? 1 : 256 / ncv; }

template <typename T>
__global__ void gn_stats_kernel(const T* __restrict__ x, float* __restrict__ sum,
                                float* __restrict__ sumsq, int HW, int C, int G, int rows) {
  extern __shared__ float chan[];       // [2][C]
  const int ncv = C / 8, cpg = C / G;
  const int cv = threadIdx.x % ncv, r = threadIdx.x / ncv;
  const int b = blockIdx.y;
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) chan[i] = 0.f;
  __syncthreads();
  const int per = (HW + gridDim.x - 1) / gridDim.x;
  const int p0 = blockIdx.x * per, p1 = min(HW, p0 + per);
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0}, q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const T* base = x + (long long)b * HW * C + cv * 8;
  for (int p = p0 + r; p < p1; p += rows) {
    const uint4 u = *reinterpret_cast<const uint4*>(base + (long long)p * C);
    const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float v = to_f32<T>(e[j]); s[j] += v; q[j] = fmaf(v, v, q[j]); }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    atomicAdd(&chan[cv * 8 + j], s[j]);
    atomicAdd(&chan[C + cv * 8 + j], q[j]);
  }
  __syncthreads();
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    float a = 0.f, c = 0.f;
    for (int i = 0; i < cpg; ++i) { a += chan[g * cpg + i]; c += chan[C + g * cpg + i]; }
    atomicAdd(&sum[b * G + g], a);
    atomicAdd(&sumsq[b * G + g], c);
  }
}

// (sum, sumsq) -> (mean, rstd), in place
__global__ void gn_finalize_kernel(float* __restrict__ mean, float* __restrict__ rstd, int n_groups,
                                   float inv_n, float eps) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_groups) return;
  const float m = mean[i] * inv_n;
  const float var = fmaxf(rstd[i] * inv_n - m * m, 0.f);
  mean[i] = m;
  rstd[i] = rsqrtf(var + eps);
}

// group of channel c0 + j for the 8 channels of one vector
__device__ __forceinline__ int gn_group(int c0, int j, int cpg) { return (c0 + j) / cpg; }

// y = act((x - mean) * rstd * gamma + beta), act = SiLU or identity
template <typename T>
__global__ void __launch_bounds__(256)
gn_apply_kernel(const T* __restrict__ x, const float* __restrict__ mean,
                const float* __restrict__ rstd, const float* __restrict__ gamma,
                const float* __restrict__ beta, T* __restrict__ y, long long total_vec, int HW,
                int C, int G, int act_silu) {
  const int ncv = C / 8, cpg = C / G;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec;
       i += gstride) {
    const int cv = (int)(i % ncv);
    const int b = (int)(i / ((long long)HW * ncv));
    const int c0 = cv * 8;
    const uint4 u = reinterpret_cast<const uint4*>(x)[i];
    const T* e = reinterpret_cast<const T*>(&u);
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int sg = b * G + gn_group(c0, j, cpg);
      float v = (to_f32<T>(e[j]) - mean[sg]) * rstd[sg] * gamma[c0 + j] + beta[c0 + j];
      if (act_silu) v = silu(v);
      oe[j] = from_f32<T>(v);
    }
    reinterpret_cast<uint4*>(y)[i] = o;
  }
}

// Backward pass 1: per-channel sums of dz and dz * xhat (dz = dy * act'(z)); they are the
// parameter gradients (dbeta, dgamma) and, weighted by gamma and folded per group, the two sums
// A = sum(dz * gamma), Bq = sum(dz * gamma * xhat) the second pass needs.
template <typename T>
__global__ void gn_bwd_stats_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                    const float* __restrict__ mean, const float* __restrict__ rstd,
                                    const float* __restrict__ gamma, const float* __restrict__ beta,
                                    float* __restrict__ sumA, float* __restrict__ sumB,
                                    float* __restrict__ dgamma, float* __restrict__ dbeta, int HW,
                                    int C, int G, int act_silu, int rows) {
  extern __shared__ float chan[];       // [2][C]: sum dz * xhat, sum dz
  const int ncv = C / 8, cpg = C / G;
  const int cv = threadIdx.x % ncv, r = threadIdx.x / ncv;
  const int b = blockIdx.y, c0 = cv * 8;
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) chan[i] = 0.f;
  __syncthreads();
  float m[8], rs[8], ga[8], be[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int sg = b * G + gn_group(c0, j, cpg);
    m[j] = mean[sg]; rs[j] = rstd[sg]; ga[j] = gamma[c0 + j]; be[j] = beta[c0 + j];
  }
  const int per = (HW + gridDim.x - 1) / gridDim.x;
  const int p0 = blockIdx.x * per, p1 = min(HW, p0 + per);
  float sx[8] = {0, 0, 0, 0, 0, 0, 0, 0}, sd[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const long long off = (long long)b * HW * C + c0;
  for (int p = p0 + r; p < p1; p += rows) {
    const uint4 ux = *reinterpret_cast<const uint4*>(x + off + (long long)p * C);
    const uint4 ud = *reinterpret_cast<const uint4*>(dy + off + (long long)p * C);
    const T* ex = reinterpret_cast<const T*>(&ux);
    const T* ed = reinterpret_cast<const T*>(&ud);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float xhat = (to_f32<T>(ex[j]) - m[j]) * rs[j];
      float dz = to_f32<T>(ed[j]);
      if (act_silu) dz *= dsilu(fmaf(xhat, ga[j], be[j]));
      sd[j] += dz;
      sx[j] = fmaf(dz, xhat, sx[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    atomicAdd(&chan[c0 + j], sx[j]);
    atomicAdd(&chan[C + c0 + j], sd[j]);
  }
  __syncthreads();
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    float a = 0.f, q = 0.f;
    for (int i = 0; i < cpg; ++i) {
      const int c = g * cpg + i;
      a = fmaf(gamma[c], chan[C + c], a);
      q = fmaf(gamma[c], chan[c], q);
    }
    atomicAdd(&sumA[b * G + g], a);
    atomicAdd(&sumB[b * G + g], q);
  }
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    atomicAdd(&dgamma[c], chan[c]);
    atomicAdd(&dbeta[c], chan[C + c]);
  }
}

// Backward pass 2: dx = rstd * (dz*gamma - A/n - xhat * B/n)
template <typename T>
__global__ void __launch_bounds__(256)
gn_bwd_apply_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                    const float* __restrict__ mean, const float* __restrict__ rstd,
                    const float* __restrict__ gamma, const float* __restrict__ beta,
                    const float* __restrict__ sumA, const float* __restrict__ sumB,
                    T* __restrict__ dx, long long total_vec, int HW, int C, int G, int act_silu) {
  const int ncv = C / 8, cpg = C / G;
  const float inv_n = 1.f / ((float)HW * cpg);
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec;
       i += gstride) {
    const int cv = (int)(i % ncv);
    const int b = (int)(i / ((long long)HW * ncv));
    const int c0 = cv * 8;
    const uint4 ux = reinterpret_cast<const uint4*>(x)[i];
    const uint4 ud = reinterpret_cast<const uint4*>(dy)[i];
    const T* ex = reinterpret_cast<const T*>(&ux);
    const T* ed = reinterpret_cast<const T*>(&ud);
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int sg = b * G + gn_group(c0, j, cpg);
      const float rs = rstd[sg];
      const float xhat = (to_f32<T>(ex[j]) - mean[sg]) * rs;
      float dz = to_f32<T>(ed[j]);
      const float g = gamma[c0 + j];
      if (act_silu) dz *= dsilu(fmaf(xhat, g, beta[c0 + j]));
      oe[j] = from_f32<T>(rs * (dz * g - sumA[sg] * inv_n - xhat * sumB[sg] * inv_n));
    }
    reinterpret_cast<uint4*>(dx)[i] = o;
  }
}

// nearest 2x upsample (NHWC) and its backward (sum of the 4 children)
template <typename T>
__global__ void __launch_bounds__(256)
upsample2x_kernel(const T* __restrict__ x, T* __restrict__ y, int B, int H, int W, int C,
                  int backward) {
  const int cv = C / 8;
  const long long total = backward ? (long long)B * H * W * cv : (long long)B * 4 * H * W * cv;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
    const int c8 = (int)(i % cv);
    long long t = i / cv;
    if (!backward) {
      const int wo = (int)(t % (2 * W)); t /= 2 * W;
      const int ho = (int)(t % (2 * H));
      const int b = (int)(t / (2 * H));
      reinterpret_cast<uint4*>(y + (((long long)b * 2 * H + ho) * 2 * W + wo) * C)[c8] =
          reinterpret_cast<const uint4*>(x + (((long long)b * H + ho / 2) * W + wo / 2) * C)[c8];
    } else {   // x = dy [B, 2H, 2W, C], y = dx [B, H, W, C]
      const int wi = (int)(t % W); t /= W;
      const int hi = (int)(t % H);
      const int b = (int)(t / H);
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int dh = 0; dh < 2; ++dh)
        for (int dw = 0; dw < 2; ++dw) {
          uint4 q = reinterpret_cast<const uint4*>(
              x + (((long long)b * 2 * H + 2 * hi + dh) * 2 * W + 2 * wi + dw) * C)[c8];
          const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += to_f32<T>(e[j]);
        }
      uint4 o;
      T* e = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(acc[j]);
      reinterpret_cast<uint4*>(y + (((long long)b * H + hi) * W + wi) * C)[c8] = o;
    }
  }
}

static inline int grid_for(long long n, int sm_count) {
  long long b = (n + 255) / 256;
  const long long cap = (long long)(sm_count > 0 ? sm_count : 148) * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace pf

using namespace pf;

#define PF_DISPATCH_H(dtype, ...)                               \
  switch (dtype) {                                             \
    case PF_F16: { using T = __half; __VA_ARGS__; } break;      \
    case PF_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break; \
    default: return -1;                                        \
  }

PF_API int pf_im2col(const void* x, void* cols, int B, int H, int W, int C, int KH, int KW, int Ho,
                     int Wo, int stride, int pad, long long ldc, int dtype, int sm_count,
                     void* stream) {
  if (C % 8 || ldc % 8) return -2;
  const long long total = (long long)B * Ho * Wo * KH * KW * (C / 8);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PF_DISPATCH_H(dtype, (im2col_kernel<T><<<grid_for(total, sm_count), 256, 0, st>>>(
      (const T*)x, (T*)cols, B, H, W, C, KH, KW, Ho, Wo, stride, pad, ldc)));
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_col2im(const void* dcols, void* dx, int B, int H, int W, int C, int KH, int KW,
                     int Ho, int Wo, int stride, int pad, long long ldc, int dtype, int sm_count,
                     void* stream) {
  if (C % 8 || ldc % 8) return -2;
  const long long total = (long long)B * H * W * (C / 8);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PF_DISPATCH_H(dtype, (col2im_kernel<T><<<grid_for(total, sm_count), 256, 0, st>>>(
      (const T*)dcols, (T*)dx, B, H, W, C, KH, KW, Ho, Wo, stride, pad, ldc)));
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_groupnorm_fwd(const void* x, const void* gamma, const void* beta, void* y,
                            void* mean, void* rstd, int B, int HW, int C, int G, float eps,
                            int act_silu, int dtype, int sm_count, void* stream) {
  if (C % G || C % 8) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long total_vec = (long long)B * HW * (C / 8);
  const int rows = gn_rows(C);
  const int threads = rows * (C / 8);
  if (threads > 1024) return -2;
  int slabs = (4 * (sm_count > 0 ? sm_count : 148) + B - 1) / B;
  if (slabs > (HW + rows - 1) / rows) slabs = (HW + rows - 1) / rows;
  if (slabs < 1) slabs = 1;
  // mean / rstd first hold the sums, then are converted in place
  cudaMemsetAsync(mean, 0, sizeof(float) * B * G, st);
  cudaMemsetAsync(rstd, 0, sizeof(float) * B * G, st);
  PF_DISPATCH_H(dtype, {
    gn_stats_kernel<T><<<dim3(slabs, B), threads, 2 * C * sizeof(float), st>>>(
        (const T*)x, (float*)mean, (float*)rstd, HW, C, G, rows);
    gn_finalize_kernel<<<(B * G + 255) / 256, 256, 0, st>>>(
        (float*)mean, (float*)rstd, B * G, 1.f / ((float)HW * (C / G)), eps);
    gn_apply_kernel<T><<<grid_for(total_vec, sm_count), 256, 0, st>>>(
        (const T*)x, (const float*)mean, (const float*)rstd, (const float*)gamma,
        (const float*)beta, (T*)y, total_vec, HW, C, G, act_silu);
  });
  PF_CHECK_LAUNCH();
  return 0;
}

// sums: fp32 scratch [2][B*G] (zeroed here); dgamma / dbeta fp32 [C], accumulated into (zero
// them first for a fresh gradient)
PF_API int pf_groupnorm_bwd(const void* dy, const void* x, const void* mean, const void* rstd,
                            const void* gamma, const void* beta, void* dx, void* dgamma,
                            void* dbeta, void* sums, int B, int HW, int C, int G, int act_silu,
                            int dtype, int sm_count, void* stream) {
  if (C % G || C % 8) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long total_vec = (long long)B * HW * (C / 8);
  float* sA = (float*)sums;
  float* sB = sA + (long long)B * G;
  const int rows = gn_rows(C);
  const int threads = rows * (C / 8);
  if (threads > 1024) return -2;
  int slabs = (4 * (sm_count > 0 ? sm_count : 148) + B - 1) / B;
  if (slabs > (HW + rows - 1) / rows) slabs = (HW + rows - 1) / rows;
  if (slabs < 1) slabs = 1;
  cudaMemsetAsync(sums, 0, sizeof(float) * 2 * B * G, st);
  PF_DISPATCH_H(dtype, {
    gn_bwd_stats_kernel<T><<<dim3(slabs, B), threads, 2 * C * sizeof(float), st>>>(
        (const T*)dy, (const T*)x, (const float*)mean, (const float*)rstd, (const float*)gamma,
        (const float*)beta, sA, sB, (float*)dgamma, (float*)dbeta, HW, C, G, act_silu, rows);
    gn_bwd_apply_kernel<T><<<grid_for(total_vec, sm_count), 256, 0, st>>>(
        (const T*)dy, (const T*)x, (const float*)mean, (const float*)rstd, (const float*)gamma,
        (const float*)beta, sA, sB, (T*)dx, total_vec, HW, C, G, act_silu);
  });
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_upsample2x(const void* x, void* y, int B, int H, int W, int C, int backward,
                         int dtype, int sm_count, void* stream) {
  if (C % 8) return -2;
  const long long total = (long long)B * H * W * (C / 8) * (backward ? 1 : 4);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PF_DISPATCH_H(dtype, (upsample2x_kernel<T><<<grid_for(total, sm_count), 256, 0, st>>>(
      (const T*)x, (T*)y, B, H, W, C, backward)));
  PF_CHECK_LAUNCH();
  return 0;
}
