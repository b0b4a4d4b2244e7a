// Optimizer-side kernels on flat buffers: non-finite check, fused unscale + AdamW (+ optional
// 16-bit shadow-weight write and gradient zeroing), SGD with momentum.
//
// The skip decision of dynamic loss scaling lives on the device: `found_inf` is a float that is
// non-zero when any gradient of the step was non-finite; the update kernels read it and leave
// parameters and moments untouched, so no host sync is needed between backward and the update.
#include "common.cuh"
#include "api.h"

namespace pf {

__global__ void __launch_bounds__(256)
nonfinite_kernel(const float* __restrict__ g, long long n, float* __restrict__ found_inf) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  bool bad = false;
  const long long nvec = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float4 v = reinterpret_cast<const float4*>(g)[i];
    bad |= !(isfinite(v.x) && isfinite(v.y) && isfinite(v.z) && isfinite(v.w));
  }
  for (long long i = nvec * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    bad |= !isfinite(g[i]);
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) *found_inf = 1.0f;
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay;
  int step;            // 1-based step number, used when no device counter is given
  float grad_scale;    // multiplies the gradient (1 / loss_scale / accumulation count)
  int adamw;           // decoupled decay (AdamW) or L2 (Adam)
  int zero_grad;
  int lp_dtype;        // dtype of the optional 16-bit shadow
};

// One pass: read g, p, m, v (fp32) -> write p, m, v, optional 16-bit shadow, optional g = 0.
// 16 B per access; 4 elements per thread per iteration.
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
             float* __restrict__ v, void* __restrict__ lp, long long n,
             const float* __restrict__ found_inf, const float* __restrict__ loss_scale,
             const int* __restrict__ applied_steps, AdamArgs a) {
  if (loss_scale) a.grad_scale /= *loss_scale;
  if (found_inf && *found_inf != 0.f) {
    if (a.zero_grad) {
      const long long stride = (long long)gridDim.x * blockDim.x;
      for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        g[i] = 0.f;
    }
    return;
  }
  const long long nvec = n / 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  // bias correction from the number of steps that were really applied: a step skipped on a
  // gradient overflow does not advance it (the counter moves after all groups were updated)
  const float t = (float)(applied_steps ? *applied_steps + 1 : a.step);
  const float inv_bc1 = 1.f / (1.f - powf(a.beta1, t));
  const float inv_sqrt_bc2 = rsqrtf(1.f - powf(a.beta2, t));
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float4 pg = reinterpret_cast<float4*>(g)[i];
    float4 pp = reinterpret_cast<float4*>(p)[i];
    float4 pm = reinterpret_cast<float4*>(m)[i];
    float4 pv = reinterpret_cast<float4*>(v)[i];
    float gg[4] = {pg.x, pg.y, pg.z, pg.w};
    float ww[4] = {pp.x, pp.y, pp.z, pp.w};
    float mm[4] = {pm.x, pm.y, pm.z, pm.w};
    float vv[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gr = gg[j] * a.grad_scale;
      if (a.adamw) ww[j] *= (1.f - a.lr * a.weight_decay);
      else gr += a.weight_decay * ww[j];
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gr;
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gr * gr;
      const float denom = sqrtf(vv[j]) * inv_sqrt_bc2 + a.eps;
      ww[j] -= a.lr * (mm[j] * inv_bc1) / denom;
    }
    reinterpret_cast<float4*>(p)[i] = make_float4(ww[0], ww[1], ww[2], ww[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (a.zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (lp) {
      if (a.lp_dtype == PF_BF16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(ww[0], ww[1]);
        __nv_bfloat162 hi = __floats2bfloat162_rn(ww[2], ww[3]);
        uint2 q = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        reinterpret_cast<uint2*>(lp)[i] = q;
      } else {
        __half2 lo = __floats2half2_rn(ww[0], ww[1]);
        __half2 hi = __floats2half2_rn(ww[2], ww[3]);
        uint2 q = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        reinterpret_cast<uint2*>(lp)[i] = q;
      }
    }
  }
  // tail
  for (long long i = nvec * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float gr = g[i] * a.grad_scale;
    float w = p[i];
    if (a.adamw) w *= (1.f - a.lr * a.weight_decay);
    else gr += a.weight_decay * w;
    const float mi = a.beta1 * m[i] + (1.f - a.beta1) * gr;
    const float vi = a.beta2 * v[i] + (1.f - a.beta2) * gr * gr;
    w -= a.lr * (mi * inv_bc1) / (sqrtf(vi) * inv_sqrt_bc2 + a.eps);
    p[i] = w; m[i] = mi; v[i] = vi;
    if (a.zero_grad) g[i] = 0.f;
    if (lp) {
      if (a.lp_dtype == PF_BF16) reinterpret_cast<__nv_bfloat16*>(lp)[i] = __float2bfloat16_rn(w);
      else reinterpret_cast<__half*>(lp)[i] = __float2half_rn(w);
    }
  }
}

__global__ void __launch_bounds__(256)
sgd_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ mom,
           void* __restrict__ lp, long long n, const float* __restrict__ found_inf, float lr,
           float momentum, float dampening, float weight_decay, int nesterov, int first_step,
           float grad_scale, int zero_grad, int lp_dtype,
           const float* __restrict__ loss_scale) {
  if (loss_scale) grad_scale /= *loss_scale;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const bool skip = found_inf && *found_inf != 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    if (!skip) {
      float gr = g[i] * grad_scale + weight_decay * p[i];
      if (mom) {
        float b = first_step ? gr : momentum * mom[i] + (1.f - dampening) * gr;
        mom[i] = b;
        gr = nesterov ? gr + momentum * b : b;
      }
      const float w = p[i] - lr * gr;
      p[i] = w;
      if (lp) {
        if (lp_dtype == PF_BF16) reinterpret_cast<__nv_bfloat16*>(lp)[i] = __float2bfloat16_rn(w);
        else reinterpret_cast<__half*>(lp)[i] = __float2half_rn(w);
      }
    }
    if (zero_grad) g[i] = 0.f;
  }
}

// applied-step counter of the Adam family: advances unless the step was skipped
__global__ void step_advance_kernel(int* applied_steps, const float* found_inf) {
  if (threadIdx.x == 0 && blockIdx.x == 0 && !(found_inf && *found_inf != 0.f)) *applied_steps += 1;
}

// scale update of dynamic loss scaling, entirely on the device:
//   state = {scale, growth_tracker}; found_inf is reset afterwards
__global__ void loss_scale_update_kernel(float* state, float* found_inf, float growth,
                                         float backoff, int interval) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    if (*found_inf != 0.f) {
      state[0] *= backoff;
      state[1] = 0.f;
    } else {
      state[1] += 1.f;
      if ((int)state[1] >= interval) {
        state[0] *= growth;
        state[1] = 0.f;
      }
    }
    *found_inf = 0.f;
  }
}

static inline int opt_grid(long long n, int sm_count) {
  long long b = (n / 4 + 255) / 256;
  long long cap = (long long)(sm_count > 0 ? sm_count : 148) * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace pf

using namespace pf;

PF_API int pf_nonfinite(const void* g, long long n, void* found_inf, int sm_count, void* stream) {
  if (n <= 0) return 0;
  nonfinite_kernel<<<opt_grid(n, sm_count), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const float*)g, n, (float*)found_inf);
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_adamw(void* p, void* g, void* m, void* v, void* lp, long long n,
                    const void* found_inf, const void* loss_scale, float lr, float beta1, float beta2, float eps,
                    float weight_decay, int step, const void* applied_steps, float grad_scale,
                    int adamw, int zero_grad, int lp_dtype, int sm_count, void* stream) {
  if (n <= 0) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.step = step;
  a.grad_scale = grad_scale; a.adamw = adamw; a.zero_grad = zero_grad; a.lp_dtype = lp_dtype;
  adamw_kernel<<<opt_grid(n, sm_count), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (float*)p, (float*)g, (float*)m, (float*)v, lp, n, (const float*)found_inf,
      (const float*)loss_scale, (const int*)applied_steps, a);
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_step_advance(void* applied_steps, const void* found_inf, void* stream) {
  step_advance_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (int*)applied_steps, (const float*)found_inf);
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_sgd(void* p, void* g, void* mom, void* lp, long long n, const void* found_inf,
                  const void* loss_scale, float lr, float momentum, float dampening, float weight_decay, int nesterov,
                  int first_step, float grad_scale, int zero_grad, int lp_dtype, int sm_count,
                  void* stream) {
  if (n <= 0) return 0;
  sgd_kernel<<<opt_grid(n, sm_count), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (float*)p, (float*)g, (float*)mom, lp, n, (const float*)found_inf, lr, momentum, dampening,
      weight_decay, nesterov, first_step, grad_scale, zero_grad, lp_dtype,
      (const float*)loss_scale);
  PF_CHECK_LAUNCH();
  return 0;
}

PF_API int pf_loss_scale_update(void* state, void* found_inf, float growth, float backoff,
                                int interval, void* stream) {
  loss_scale_update_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (float*)state, (float*)found_inf, growth, backoff, interval);
  PF_CHECK_LAUNCH();
  return 0;
}
