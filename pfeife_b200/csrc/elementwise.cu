// Vectorised elementwise kernels (stand-alone forms of the activations that are not fused into
// a GEMM epilogue), casts, transposes, column sums and stage-boundary pack/accumulate.
// All of them move 16 bytes per thread per access and are bound by HBM bandwidth.
#include "common.cuh"
#include "api.h"

namespace pf {

constexpr int EW_THREADS = 256;

static inline int ew_grid(long long nvec, int sm_count) {
  long long blocks = (nvec + EW_THREADS - 1) / EW_THREADS;
  long long cap = (long long)(sm_count > 0 ? sm_count : 148) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  uint4 q;
  __device__ __forceinline__ float get(int i) const {
    return to_f32<T>(reinterpret_cast<const T*>(&q)[i]);
  }
  __device__ __forceinline__ void set(int i, float v) {
    reinterpret_cast<T*>(&q)[i] = from_f32<T>(v);
  }
};

// op codes for the unary / binary family
enum EwOp : int {
  EW_GELU = 0, EW_GELU_TANH = 1, EW_SILU = 2, EW_COPY = 3,
  EW_DGELU = 10, EW_DGELU_TANH = 11, EW_DSILU = 12,  // out = a(dy) * f'(b(x))
  EW_ADD = 20, EW_MUL = 21,
  EW_SILU_MUL = 30,                                   // out = silu(a) * b
  EW_GELU_MUL = 31,                                   // out = gelu(a) * b   (GEGLU)
};

template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
ew_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, long long n,
          int op) {
  constexpr int V = Vec16<T>::N;
  const long long nvec = n / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Vec16<T> va, vb, vo;
    va.q = reinterpret_cast<const uint4*>(a)[i];
    if (b) vb.q = reinterpret_cast<const uint4*>(b)[i];
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float x = va.get(j);
      const float y = b ? vb.get(j) : 0.f;
      float r;
      switch (op) {
        case EW_GELU: r = gelu_erf(x); break;
        case EW_GELU_TANH: r = gelu_tanh(x); break;
        case EW_SILU: r = silu(x); break;
        case EW_DGELU: r = x * dgelu_erf(y); break;
        case EW_DGELU_TANH: r = x * dgelu_tanh(y); break;
        case EW_DSILU: r = x * dsilu(y); break;
        case EW_ADD: r = x + y; break;
        case EW_MUL: r = x * y; break;
        case EW_SILU_MUL: r = silu(x) * y; break;
        case EW_GELU_MUL: r = gelu_erf(x) * y; break;
        default: r = x;
      }
      vo.set(j, r);
    }
    reinterpret_cast<uint4*>(out)[i] = vo.q;
  }
  // tail (n not a multiple of the vector width)
  const long long tail0 = nvec * V;
  for (long long i = tail0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float x = to_f32<T>(a[i]);
    const float y = b ? to_f32<T>(b[i]) : 0.f;
    float r;
    switch (op) {
      case EW_GELU: r = gelu_erf(x); break;
      case EW_GELU_TANH: r = gelu_tanh(x); break;
      case EW_SILU: r = silu(x); break;
      case EW_DGELU: r = x * dgelu_erf(y); break;
      case EW_DGELU_TANH: r = x * dgelu_tanh(y); break;
      case EW_DSILU: r = x * dsilu(y); break;
      case EW_ADD: r = x + y; break;
      case EW_MUL: r = x * y; break;
      case EW_SILU_MUL: r = silu(x) * y; break;
      case EW_GELU_MUL: r = gelu_erf(x) * y; break;
      default: r = x;
    }
    out[i] = from_f32<T>(r);
  }
}

// Gated activations on a fused [rows, 2*H] projection (gate = cols [0,H), up = cols [H,2H)):
//   out[r, h] = act(gate) * up          (SwiGLU: act = silu, GEGLU: act = gelu)
// and their backward, which writes d(gate|up) back in the fused layout.
template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
glu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int H, int gelu) {
  constexpr int V = Vec16<T>::N;
  const int hv = H / V;
  const long long total = rows * hv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / hv;
    const int c = (int)(i - r * hv);
    Vec16<T> g, u, o;
    g.q = reinterpret_cast<const uint4*>(gu + r * 2 * H)[c];
    u.q = reinterpret_cast<const uint4*>(gu + r * 2 * H + H)[c];
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float x = g.get(j);
      o.set(j, (gelu ? gelu_erf(x) : silu(x)) * u.get(j));
    }
    reinterpret_cast<uint4*>(out + r * H)[c] = o.q;
  }
}

template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
glu_bwd_kernel(const T* __restrict__ gu, const T* __restrict__ dout, T* __restrict__ dgu,
               long long rows, int H, int gelu) {
  constexpr int V = Vec16<T>::N;
  const int hv = H / V;
  const long long total = rows * hv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / hv;
    const int c = (int)(i - r * hv);
    Vec16<T> g, u, d, dg, du;
    g.q = reinterpret_cast<const uint4*>(gu + r * 2 * H)[c];
    u.q = reinterpret_cast<const uint4*>(gu + r * 2 * H + H)[c];
    d.q = reinterpret_cast<const uint4*>(dout + r * H)[c];
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float x = g.get(j), y = u.get(j), dy = d.get(j);
      const float a = gelu ? gelu_erf(x) : silu(x);
      const float da = gelu ? dgelu_erf(x) : dsilu(x);
      dg.set(j, dy * y * da);
      du.set(j, dy * a);
    }
    reinterpret_cast<uint4*>(dgu + r * 2 * H)[c] = dg.q;
    reinterpret_cast<uint4*>(dgu + r * 2 * H + H)[c] = du.q;
  }
}

// dst(fp32) (+)= src(T) * scale : receive-side accumulate of several gradient buffers, and the
// hand-off of 16-bit gradients into fp32 buckets.
template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
axpy_f32_kernel(float* __restrict__ dst, const T* __restrict__ src, long long n, float scale,
                int accumulate) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = to_f32<T>(src[i]) * scale;
    dst[i] = accumulate ? dst[i] + v : v;
  }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(EW_THREADS)
cast_kernel(const TI* __restrict__ src, TO* __restrict__ dst, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = from_f32<TO>(to_f32<TI>(src[i]));
}

// out[c] (+)= sum_r x[r, c]   (bias gradients).  Each CTA owns 32 columns x a slab of rows and
// finishes with one atomicAdd per column, so `out` must be zeroed (or hold the running
// gradient) before the launch.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_kernel(const T* __restrict__ x, float* __restrict__ out, long long rows, int cols,
              long long ld, int rows_per_cta) {
  __shared__ float part[8][33];
  const int c = blockIdx.x * 32 + (threadIdx.x & 31);
  const int ry = threadIdx.x >> 5;
  const long long r0 = (long long)blockIdx.y * rows_per_cta;
  const long long r1 = min(rows, r0 + rows_per_cta);
  float s = 0.f;
  if (c < cols)
    for (long long r = r0 + ry; r < r1; r += 8) s += to_f32<T>(x[r * ld + c]);
  part[ry][threadIdx.x & 31] = s;
  __syncthreads();
  if (ry == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += part[i][threadIdx.x];
    atomicAdd(out + c, t);
  }
}

// Same reduction for 16-bit inputs whose pitch allows 16-byte loads: a CTA owns 256 columns
// (lane = 8 consecutive columns) and a slab of rows split over its 8 warps.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_vec_kernel(const T* __restrict__ x, float* __restrict__ out, long long rows, int cols,
                  long long ld, int rows_per_cta) {
  __shared__ float red[8][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 256 + lane * 8;
  const long long r0 = (long long)blockIdx.y * rows_per_cta;
  const long long r1 = min(rows, r0 + rows_per_cta);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c0 < cols) {
    for (long long r = r0 + warp; r < r1; r += 8) {
      const uint4 q = *reinterpret_cast<const uint4*>(x + r * ld + c0);
      const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += to_f32<T>(e[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = acc[j];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < cols) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][threadIdx.x];
    atomicAdd(out + c, t);
  }
}

// 16-bit tiled transpose: dst[c, r] = src[r, c]
template <typename T>
__global__ void __launch_bounds__(256)
transpose_kernel(const T* __restrict__ src, T* __restrict__ dst, int rows, int cols,
                 long long ld_src, long long ld_dst) {
  __shared__ T tile[32][33];
  const int bx = blockIdx.x * 32, by = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int j = ty; j < 32; j += 8) {
    const int r = by + j, c = bx + tx;
    if (r < rows && c < cols) tile[j][tx] = src[(long long)r * ld_src + c];
  }
  __syncthreads();
#pragma unroll
  for (int j = ty; j < 32; j += 8) {
    const int c = bx + j, r = by + tx;
    if (r < rows && c < cols) dst[(long long)c * ld_dst + r] = tile[tx][j];
  }
}

}  // namespace pf

using namespace pf;

#define PF_DISPATCH_16_32(dtype, ...)                          \
  switch (dtype) {                                             \
    case PF_F32: { using T = float; __VA_ARGS__; } break;       \
    case PF_F16: { using T = __half; __VA_ARGS__; } break;      \
    case PF_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break; \
    default: return -1;                                        \
  }

PF_API int pf_elementwise(const void* a, const void* b, void* out, long long n, int op, int dtype,
                          int sm_count, void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PF_DISPATCH_16_32(dtype, {
    const long long nvec = n / Vec16<T>::N + 1;
    ew_kernel<T><<<ew_grid(nvec, sm_count), EW_THREADS, 0, st>>>(
        (const T*)a, (const T*)b, (T*)out, n, op);
  });
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_glu_fwd(const void* gu, void* out, long long rows, int H, int gelu, int dtype,
                      int sm_count, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PF_DISPATCH_16_32(dtype, {
    if (H % Vec16<T>::N) return -2;
    const long long total = rows * (H / Vec16<T>::N);
    glu_fwd_kernel<T><<<ew_grid(total, sm_count), EW_THREADS, 0, st>>>((const T*)gu, (T*)out,
                                                                       rows, H, gelu);
  });
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_glu_bwd(const void* gu, const void* dout, void* dgu, long long rows, int H, int gelu,
                      int dtype, int sm_count, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PF_DISPATCH_16_32(dtype, {
    if (H % Vec16<T>::N) return -2;
    const long long total = rows * (H / Vec16<T>::N);
    glu_bwd_kernel<T><<<ew_grid(total, sm_count), EW_THREADS, 0, st>>>(
        (const T*)gu, (const T*)dout, (T*)dgu, rows, H, gelu);
  });
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_axpy_f32(void* dst, const void* src, long long n, float scale, int accumulate,
                       int src_dtype, int sm_count, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PF_DISPATCH_16_32(src_dtype, {
    axpy_f32_kernel<T><<<ew_grid(n, sm_count), EW_THREADS, 0, st>>>((float*)dst, (const T*)src, n,
                                                                    scale, accumulate);
  });
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_cast(const void* src, void* dst, long long n, int src_dtype, int dst_dtype,
                   int sm_count, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int g = ew_grid(n, sm_count);
#define PF_CAST_CASE(SD, ST, DD, DT) \
  if (src_dtype == SD && dst_dtype == DD) cast_kernel<ST, DT><<<g, EW_THREADS, 0, st>>>((const ST*)src, (DT*)dst, n);
  PF_CAST_CASE(PF_F32, float, PF_F16, __half)
  else PF_CAST_CASE(PF_F32, float, PF_BF16, __nv_bfloat16)
  else PF_CAST_CASE(PF_F16, __half, PF_F32, float)
  else PF_CAST_CASE(PF_BF16, __nv_bfloat16, PF_F32, float)
  else PF_CAST_CASE(PF_F32, float, PF_F32, float)
  else PF_CAST_CASE(PF_F16, __half, PF_F16, __half)
  else PF_CAST_CASE(PF_BF16, __nv_bfloat16, PF_BF16, __nv_bfloat16)
  else PF_CAST_CASE(PF_F16, __half, PF_BF16, __nv_bfloat16)
  else PF_CAST_CASE(PF_BF16, __nv_bfloat16, PF_F16, __half)
  else return -1;
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_colsum(const void* x, void* out_f32, long long rows, int cols, long long ld,
                     int dtype, int sm_count, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype != PF_F32 && cols % 8 == 0 && ld % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int gxv = (cols + 255) / 256;
    int gyv = ((sm_count > 0 ? sm_count : 148) * 4 + gxv - 1) / gxv;
    int per = (int)((rows + gyv - 1) / gyv);
    if (per < 32) per = 32;
    gyv = (int)((rows + per - 1) / per);
    if (dtype == PF_F16)
      colsum_vec_kernel<__half><<<dim3(gxv, gyv), 256, 0, st>>>((const __half*)x, (float*)out_f32,
                                                                rows, cols, ld, per);
    else
      colsum_vec_kernel<__nv_bfloat16><<<dim3(gxv, gyv), 256, 0, st>>>(
          (const __nv_bfloat16*)x, (float*)out_f32, rows, cols, ld, per);
    PF_CHECK_LAUNCH();
    return 0;
  }
  const int gx = (cols + 31) / 32;
  int gy = ((sm_count > 0 ? sm_count : 148) * 4 + gx - 1) / gx;
  if (gy < 1) gy = 1;
  int rows_per = (int)((rows + gy - 1) / gy);
  if (rows_per < 64) rows_per = 64;
  gy = (int)((rows + rows_per - 1) / rows_per);
  PF_DISPATCH_16_32(dtype, {
    colsum_kernel<T><<<dim3(gx, gy), 256, 0, st>>>((const T*)x, (float*)out_f32, rows, cols, ld,
                                                   rows_per);
  });
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_transpose16(const void* src, void* dst, int rows, int cols, long long ld_src,
                          long long ld_dst, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((cols + 31) / 32, (rows + 31) / 32);
  transpose_kernel<__half><<<grid, 256, 0, st>>>((const __half*)src, (__half*)dst, rows, cols,
                                                 ld_src, ld_dst);
  PF_CHECK_LAUNCH();
  return 0;
}
