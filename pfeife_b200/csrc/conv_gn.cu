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
// stats[b, g] = (mean, rstd) over HW x (C/G) elements.  One CTA per (b, g).
template <typename T>
__global__ void __launch_bounds__(256)
gn_stats_kernel(const T* __restrict__ x, float* __restrict__ mean, float* __restrict__ rstd,
                int HW, int C, int G, float eps) {
  __shared__ float red[2][8];
  const int b = blockIdx.x / G, g = blockIdx.x % G;
  const int cpg = C / G;
  const T* base = x + (long long)b * HW * C + g * cpg;
  const long long n = (long long)HW * cpg;
  float s = 0.f, ss = 0.f;
  for (long long i = threadIdx.x; i < n; i += 256) {
    const long long p = i / cpg;
    const int c = (int)(i - p * cpg);
    const float v = to_f32<T>(base[p * C + c]);
    s += v; ss += v * v;
  }
  s = warp_sum(s); ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = s; red[1][threadIdx.x >> 5] = ss; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, q = 0.f;
    for (int i = 0; i < 8; ++i) { a += red[0][i]; q += red[1][i]; }
    const float m = a / n;
    const float var = fmaxf(q / n - m * m, 0.f);
    mean[blockIdx.x] = m;
    rstd[blockIdx.x] = rsqrtf(var + eps);
  }
}

// y = act((x - mean) * rstd * gamma + beta), act = SiLU or identity; elementwise over NHWC
template <typename T>
__global__ void __launch_bounds__(256)
gn_apply_kernel(const T* __restrict__ x, const float* __restrict__ mean,
                const float* __restrict__ rstd, const float* __restrict__ gamma,
                const float* __restrict__ beta, T* __restrict__ y, long long total, int HW, int C,
                int G, int act_silu) {
  const int cpg = C / G;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
    const int c = (int)(i % C);
    const long long b = i / ((long long)HW * C);
    const int sg = (int)(b * G + c / cpg);
    float v = (to_f32<T>(x[i]) - mean[sg]) * rstd[sg] * gamma[c] + beta[c];
    if (act_silu) v = silu(v);
    y[i] = from_f32<T>(v);
  }
}

// Backward pass 1: per (b, g) sums  A = sum(dz * gamma), Bq = sum(dz * gamma * xhat), and the
// parameter gradients dgamma[c] += sum dz * xhat, dbeta[c] += sum dz  (dz = dy * act'(z)).
template <typename T>
__global__ void __launch_bounds__(256)
gn_bwd_stats_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                    const float* __restrict__ mean, const float* __restrict__ rstd,
                    const float* __restrict__ gamma, const float* __restrict__ beta,
                    float* __restrict__ sumA, float* __restrict__ sumB,
                    float* __restrict__ dgamma, float* __restrict__ dbeta, int HW, int C, int G,
                    int act_silu) {
  __shared__ float red[2][8];
  extern __shared__ float chan[];   // [2][cpg]
  const int b = blockIdx.x / G, g = blockIdx.x % G;
  const int cpg = C / G;
  for (int i = threadIdx.x; i < 2 * cpg; i += 256) chan[i] = 0.f;
  __syncthreads();
  const long long off = (long long)b * HW * C + g * cpg;
  const float m = mean[blockIdx.x], rs = rstd[blockIdx.x];
  const long long n = (long long)HW * cpg;
  float a = 0.f, q = 0.f;
  for (long long i = threadIdx.x; i < n; i += 256) {
    const long long p = i / cpg;
    const int c = (int)(i - p * cpg);
    const int ch = g * cpg + c;
    const float xhat = (to_f32<T>(x[off + p * C + c]) - m) * rs;
    float dz = to_f32<T>(dy[off + p * C + c]);
    if (act_silu) dz *= dsilu(xhat * gamma[ch] + beta[ch]);
    a += dz * gamma[ch];
    q += dz * gamma[ch] * xhat;
    atomicAdd(&chan[c], dz * xhat);
    atomicAdd(&chan[cpg + c], dz);
  }
  a = warp_sum(a); q = warp_sum(q);
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = a; red[1][threadIdx.x >> 5] = q; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s0 = 0.f, s1 = 0.f;
    for (int i = 0; i < 8; ++i) { s0 += red[0][i]; s1 += red[1][i]; }
    sumA[blockIdx.x] = s0;
    sumB[blockIdx.x] = s1;
  }
  for (int i = threadIdx.x; i < cpg; i += 256) {
    atomicAdd(&dgamma[g * cpg + i], chan[i]);
    atomicAdd(&dbeta[g * cpg + i], chan[cpg + i]);
  }
}

// Backward pass 2: dx = rstd * (dz*gamma - A/n - xhat * B/n)
template <typename T>
__global__ void __launch_bounds__(256)
gn_bwd_apply_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                    const float* __restrict__ mean, const float* __restrict__ rstd,
                    const float* __restrict__ gamma, const float* __restrict__ beta,
                    const float* __restrict__ sumA, const float* __restrict__ sumB,
                    T* __restrict__ dx, long long total, int HW, int C, int G, int act_silu) {
  const int cpg = C / G;
  const float inv_n = 1.f / ((float)HW * cpg);
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
    const int c = (int)(i % C);
    const long long b = i / ((long long)HW * C);
    const int sg = (int)(b * G + c / cpg);
    const float rs = rstd[sg];
    const float xhat = (to_f32<T>(x[i]) - mean[sg]) * rs;
    float dz = to_f32<T>(dy[i]);
    if (act_silu) dz *= dsilu(xhat * gamma[c] + beta[c]);
    dx[i] = from_f32<T>(rs * (dz * gamma[c] - sumA[sg] * inv_n - xhat * sumB[sg] * inv_n));
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
  if (C % G) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long total = (long long)B * HW * C;
  PF_DISPATCH_H(dtype, {
    gn_stats_kernel<T><<<B * G, 256, 0, st>>>((const T*)x, (float*)mean, (float*)rstd, HW, C, G,
                                              eps);
    gn_apply_kernel<T><<<grid_for(total, sm_count), 256, 0, st>>>(
        (const T*)x, (const float*)mean, (const float*)rstd, (const float*)gamma,
        (const float*)beta, (T*)y, total, HW, C, G, act_silu);
  });
  PF_CHECK_LAUNCH();
  return 0;
}

// sums: fp32 scratch [2][B*G]; dgamma / dbeta fp32 [C], accumulated into (zero them first for a
// fresh gradient)
PF_API int pf_groupnorm_bwd(const void* dy, const void* x, const void* mean, const void* rstd,
                            const void* gamma, const void* beta, void* dx, void* dgamma,
                            void* dbeta, void* sums, int B, int HW, int C, int G, int act_silu,
                            int dtype, int sm_count, void* stream) {
  if (C % G) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long total = (long long)B * HW * C;
  float* sA = (float*)sums;
  float* sB = sA + (long long)B * G;
  const int cpg = C / G;
  PF_DISPATCH_H(dtype, {
    gn_bwd_stats_kernel<T><<<B * G, 256, 2 * cpg * sizeof(float), st>>>(
        (const T*)dy, (const T*)x, (const float*)mean, (const float*)rstd, (const float*)gamma,
        (const float*)beta, sA, sB, (float*)dgamma, (float*)dbeta, HW, C, G, act_silu);
    gn_bwd_apply_kernel<T><<<grid_for(total, sm_count), 256, 0, st>>>(
        (const T*)dy, (const T*)x, (const float*)mean, (const float*)rstd, (const float*)gamma,
        (const float*)beta, sA, sB, (T*)dx, total, HW, C, G, act_silu);
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
