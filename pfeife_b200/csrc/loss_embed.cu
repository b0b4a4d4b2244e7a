// Softmax cross-entropy (fused log-softmax + NLL, forward and backward), MSE, embedding
// gather / scatter-add, and rotary position embedding.
#include "common.cuh"
#include "api.h"

namespace pf {

// One CTA per row of logits.  Pass 1: running max and sum-of-exp (online).  The per-row
// log-sum-exp is saved so the backward never re-reduces.  loss[row] = lse - x[target]
// (0 for ignore_index rows).
template <typename T>
__global__ void __launch_bounds__(256)
ce_fwd_kernel(const T* __restrict__ logits, const long long* __restrict__ target,
              float* __restrict__ loss, float* __restrict__ lse, int V, long long ld,
              long long ignore_index) {
  __shared__ float smax[8], ssum[8];
  const long long row = blockIdx.x;
  const T* x = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < V; i += 256) {
    const float v = to_f32<T>(x[i]);
    if (v > m) { s = s * __expf(m - v) + 1.f; m = v; }
    else s += __expf(v - m);
  }
  // warp reduce (max, sum) pairs
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mm = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
    m = mm;
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { smax[w] = m; ssum[w] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float M = smax[0], S = ssum[0];
    for (int i = 1; i < 8; ++i) {
      const float mm = fmaxf(M, smax[i]);
      S = (M == -INFINITY ? 0.f : S * __expf(M - mm)) +
          (smax[i] == -INFINITY ? 0.f : ssum[i] * __expf(smax[i] - mm));
      M = mm;
    }
    const float L = M + logf(S);
    lse[row] = L;
    const long long t = target[row];
    loss[row] = (t == ignore_index || t < 0 || t >= V) ? 0.f : L - to_f32<T>(x[t]);
  }
}

// dlogits[row, i] = (exp(x - lse) - [i == target]) * gscale[row]
// gscale = upstream gradient per row (already divided by the number of valid rows for 'mean').
template <typename T>
__global__ void __launch_bounds__(256)
ce_bwd_kernel(const T* __restrict__ logits, const long long* __restrict__ target,
              const float* __restrict__ lse, const float* __restrict__ gscale,
              T* __restrict__ dlogits, int V, long long ld, long long ignore_index) {
  const long long row = blockIdx.x;
  const T* x = logits + row * ld;
  T* d = dlogits + row * ld;
  const long long t = target[row];
  const float g = (t == ignore_index) ? 0.f : gscale[row];
  const float L = lse[row];
  for (int i = threadIdx.x; i < V; i += 256) {
    float p = __expf(to_f32<T>(x[i]) - L);
    if (i == t) p -= 1.f;
    d[i] = from_f32<T>(p * g);
  }
}

// MSE: per-CTA partial sums of (a-b)^2 in fp32 -> atomicAdd into out[0]; backward elementwise.
template <typename T>
__global__ void __launch_bounds__(256)
mse_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b, float* __restrict__ out,
               long long n, float inv_n) {
  __shared__ float red[8];
  float s = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float d = to_f32<T>(a[i]) - to_f32<T>(b[i]);
    s += d * d;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    atomicAdd(out, t * inv_n);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
mse_bwd_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ gout,
               T* __restrict__ da, long long n, float two_inv_n) {
  const float g = gout[0] * two_inv_n;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    da[i] = from_f32<T>((to_f32<T>(a[i]) - to_f32<T>(b[i])) * g);
}

// Embedding gather: out[t, :] = table[ids[t], :]   (table fp32 or 16-bit -> out T)
template <typename TT, typename T>
__global__ void __launch_bounds__(256)
embed_fwd_kernel(const TT* __restrict__ table, const long long* __restrict__ ids,
                 T* __restrict__ out, int D, long long vocab) {
  const long long t = blockIdx.x;
  long long id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  for (int i = threadIdx.x; i < D; i += 256)
    out[t * D + i] = from_f32<T>(to_f32<TT>(table[id * D + i]));
}

// Embedding scatter-add into an fp32 gradient table
template <typename T>
__global__ void __launch_bounds__(256)
embed_bwd_kernel(const T* __restrict__ dout, const long long* __restrict__ ids,
                 float* __restrict__ dtable, int D, long long vocab) {
  const long long t = blockIdx.x;
  const long long id = ids[t];
  if (id < 0 || id >= vocab) return;
  for (int i = threadIdx.x; i < D; i += 256)
    atomicAdd(dtable + id * D + i, to_f32<T>(dout[t * D + i]));
}

// Rotary embedding on a (possibly strided) x[B, S, H, D] (half-split convention: pairs
// (i, i + D/2)) into a contiguous output.  inverse != 0 applies the transpose rotation (the backward).
// Rotary embedding, 16 bytes per access: a thread rotates 8 consecutive pairs (x[d], x[d+D/2]),
// d = 8 * v .. 8 * v + 7.  Needs D/2 a multiple of 8 and 16-byte aligned rows.
template <typename T>
__global__ void __launch_bounds__(256)
rope_vec_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ cos_t,
                const float* __restrict__ sin_t, long long B, int S, int H, int D,
                long long stride_b, long long stride_s, long long stride_h, int inverse) {
  const int half = D / 2, hv = half / 8;
  const long long total = B * S * H * hv;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
    const int v = (int)(i % hv);
    long long r = i / hv;
    const int h = (int)(r % H); r /= H;
    const int s = (int)(r % S);
    const long long b = r / S;
    const T* src = x + b * stride_b + (long long)s * stride_s + (long long)h * stride_h + v * 8;
    const uint4 u1 = *reinterpret_cast<const uint4*>(src);
    const uint4 u2 = *reinterpret_cast<const uint4*>(src + half);
    const float4* cp = reinterpret_cast<const float4*>(cos_t + (long long)s * half + v * 8);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + (long long)s * half + v * 8);
    const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const T* e1 = reinterpret_cast<const T*>(&u1);
    const T* e2 = reinterpret_cast<const T*>(&u2);
    uint4 o1, o2;
    T* q1 = reinterpret_cast<T*>(&o1);
    T* q2 = reinterpret_cast<T*>(&o2);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float x1 = to_f32<T>(e1[j]), x2 = to_f32<T>(e2[j]);
      const float sj = inverse ? -sn[j] : sn[j];
      q1[j] = from_f32<T>(x1 * c[j] - x2 * sj);
      q2[j] = from_f32<T>(x2 * c[j] + x1 * sj);
    }
    // the output is always contiguous [B, S, H, D]
    T* dst = out + ((b * S + s) * H + h) * (long long)D + v * 8;
    *reinterpret_cast<uint4*>(dst) = o1;
    *reinterpret_cast<uint4*>(dst + half) = o2;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
rope_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ cos_t,
            const float* __restrict__ sin_t, long long B, int S, int H, int D,
            long long stride_b, long long stride_s, long long stride_h, int inverse) {
  const int half = D / 2;
  const long long total = B * S * H * half;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gstride) {
    const int d = (int)(i % half);
    long long r = i / half;
    const int h = (int)(r % H); r /= H;
    const int s = (int)(r % S);
    const long long b = r / S;
    const long long off = b * stride_b + (long long)s * stride_s + (long long)h * stride_h;
    const float c = cos_t[s * half + d];
    float sn = sin_t[s * half + d];
    if (inverse) sn = -sn;
    const float x1 = to_f32<T>(x[off + d]);
    const float x2 = to_f32<T>(x[off + d + half]);
    // the output is always contiguous [B, S, H, D]
    const long long oo = ((b * S + s) * H + h) * (long long)D;
    out[oo + d] = from_f32<T>(x1 * c - x2 * sn);
    out[oo + d + half] = from_f32<T>(x2 * c + x1 * sn);
  }
}

}  // namespace pf

using namespace pf;

#define PF_DISPATCH3(dtype, ...)                               \
  switch (dtype) {                                             \
    case PF_F32: { using T = float; __VA_ARGS__; } break;       \
    case PF_F16: { using T = __half; __VA_ARGS__; } break;      \
    case PF_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break; \
    default: return -1;                                        \
  }

PF_API int pf_ce_fwd(const void* logits, const void* target, void* loss, void* lse, long long rows,
                     int V, long long ld, long long ignore_index, int dtype, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PF_DISPATCH3(dtype, (ce_fwd_kernel<T><<<(unsigned)rows, 256, 0, st>>>(
      (const T*)logits, (const long long*)target, (float*)loss, (float*)lse, V, ld, ignore_index)));
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_ce_bwd(const void* logits, const void* target, const void* lse, const void* gscale,
                     void* dlogits, long long rows, int V, long long ld, long long ignore_index,
                     int dtype, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PF_DISPATCH3(dtype, (ce_bwd_kernel<T><<<(unsigned)rows, 256, 0, st>>>(
      (const T*)logits, (const long long*)target, (const float*)lse, (const float*)gscale,
      (T*)dlogits, V, ld, ignore_index)));
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_mse_fwd(const void* a, const void* b, void* out_f32, long long n, int dtype,
                      int sm_count, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaMemsetAsync(out_f32, 0, sizeof(float), st);
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  const long long cap = (long long)(sm_count > 0 ? sm_count : 148) * 8;
  if (blocks > cap) blocks = cap;
  PF_DISPATCH3(dtype, (mse_fwd_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(
      (const T*)a, (const T*)b, (float*)out_f32, n, 1.0f / (float)n)));
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_mse_bwd(const void* a, const void* b, const void* gout_f32, void* da, long long n,
                      int dtype, int sm_count, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  long long blocks = (n + 255) / 256;
  const long long cap = (long long)(sm_count > 0 ? sm_count : 148) * 8;
  if (blocks > cap) blocks = cap;
  PF_DISPATCH3(dtype, (mse_bwd_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(
      (const T*)a, (const T*)b, (const float*)gout_f32, (T*)da, n, 2.0f / (float)n)));
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_embed_fwd(const void* table, const void* ids, void* out, long long tokens, int D,
                        long long vocab, int table_dtype, int out_dtype, void* stream) {
  if (tokens <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long* I = (const long long*)ids;
#define PF_EMB(TD, TT_, OD, OT_) \
  if (table_dtype == TD && out_dtype == OD) embed_fwd_kernel<TT_, OT_><<<(unsigned)tokens, 256, 0, st>>>((const TT_*)table, I, (OT_*)out, D, vocab);
  PF_EMB(PF_F32, float, PF_F32, float)
  else PF_EMB(PF_F32, float, PF_F16, __half)
  else PF_EMB(PF_F32, float, PF_BF16, __nv_bfloat16)
  else PF_EMB(PF_F16, __half, PF_F16, __half)
  else PF_EMB(PF_BF16, __nv_bfloat16, PF_BF16, __nv_bfloat16)
  else return -1;
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_embed_bwd(const void* dout, const void* ids, void* dtable_f32, long long tokens,
                        int D, long long vocab, int dtype, void* stream) {
  if (tokens <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PF_DISPATCH3(dtype, (embed_bwd_kernel<T><<<(unsigned)tokens, 256, 0, st>>>(
      (const T*)dout, (const long long*)ids, (float*)dtable_f32, D, vocab)));
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_rope(const void* x, void* out, const void* cos_t, const void* sin_t, long long B,
                   int S, int H, int D, long long stride_b, long long stride_s,
                   long long stride_h, int inverse, int dtype, int sm_count, void* stream) {
  const long long total = B * S * H * (D / 2);
  if (total <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long cap = (long long)(sm_count > 0 ? sm_count : 148) * 8;
  const bool vec = dtype != PF_F32 && D % 16 == 0 && stride_b % 8 == 0 && stride_s % 8 == 0 &&
                   stride_h % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(cos_t) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(sin_t) & 15) == 0;
  if (vec) {
    long long vblocks = (total / 8 + 255) / 256;
    if (vblocks > cap) vblocks = cap;
    if (vblocks < 1) vblocks = 1;
    switch (dtype) {
      case PF_F16:
        rope_vec_kernel<__half><<<(unsigned)vblocks, 256, 0, st>>>(
            (const __half*)x, (__half*)out, (const float*)cos_t, (const float*)sin_t, B, S, H, D,
            stride_b, stride_s, stride_h, inverse);
        break;
      default:
        rope_vec_kernel<__nv_bfloat16><<<(unsigned)vblocks, 256, 0, st>>>(
            (const __nv_bfloat16*)x, (__nv_bfloat16*)out, (const float*)cos_t,
            (const float*)sin_t, B, S, H, D, stride_b, stride_s, stride_h, inverse);
    }
    PF_CHECK_LAUNCH();
    return 0;
  }
  long long blocks = (total + 255) / 256;
  if (blocks > cap) blocks = cap;
  PF_DISPATCH3(dtype, (rope_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(
      (const T*)x, (T*)out, (const float*)cos_t, (const float*)sin_t, B, S, H, D, stride_b,
      stride_s, stride_h, inverse)));
  PF_CHECK_LAUNCH();
  return 0;
}
