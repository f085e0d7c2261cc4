// Optimizer kernels over flat parameter ranges: Adam with decoupled weight decay, SGD with momentum,
// the global gradient L2 norm (deterministic two-stage reduction) and the clip coefficient.
//
// The whole clip + update sequence stays on the device: the norm kernels leave
// {norm, clip scale, finite flag} in a 4-float control block that the update kernels read, so no
// gradient ever travels to the host (the reference downloads every gradient for the norm and runs
// ~14 elementwise launches per parameter: lib/core/optim/grad_utils.dart:14-48, lib/core/optim/adam.dart:41-111).
#include "common/host.h"
#include "common/reduce.cuh"

namespace dptb {

constexpr int kOptThreads = 256;

// ctrl[0] = total norm, ctrl[1] = scale applied to gradients, ctrl[2] = 1 if the norm is finite, ctrl[3] = sum of squares.
template <typename TG>
__global__ void __launch_bounds__(kOptThreads)
sqnorm_partial_kernel(const TG* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float scratch[33];
  float s = 0.0f;
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  const long long nv = n / 8 * 8;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < nv; i += stride) {
    float v[8];
    Vec8<TG>::load(g + i, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += v[j] * v[j];
  }
  if (blockIdx.x == 0)
    for (long long i = nv + threadIdx.x; i < n; i += blockDim.x) {
      const float v = to_f32(g[i]);
      s += v * v;
    }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// Sums `nparts` partials (fixed order), optionally adds a previous sum of squares (ctrl[3], for norms spanning several
// ranges), and writes the control block.  max_norm <= 0 disables clipping (scale = 1).
__global__ void __launch_bounds__(1024)
clip_finalize_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ ctrl, float max_norm,
                     int add_previous) {
  __shared__ float scratch[33];
  float s = 0.0f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) {
    if (add_previous) s += ctrl[3];
    const float total = sqrtf(s);
    const bool finite = isfinite(total);
    float scale = 1.0f;
    // Same rule as the reference: no scaling when the norm is zero, within bounds, or not finite.
    if (finite && max_norm > 0.0f && total > max_norm) scale = max_norm / total;
    ctrl[0] = total;
    ctrl[1] = scale;
    ctrl[2] = finite ? 1.0f : 0.0f;
    ctrl[3] = s;
  }
}

// g *= ctrl[1]  (only used when a caller wants clipped gradients materialised).
template <typename TG>
__global__ void __launch_bounds__(kOptThreads)
scale_by_ctrl_kernel(TG* __restrict__ g, long long n, const float* __restrict__ ctrl) {
  const float sc = ctrl[1];
  if (sc == 1.0f) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    g[i] = from_f32<TG>(to_f32(g[i]) * sc);
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2;
  int skip_if_nonfinite;
  // Optional device-resident {lr, bias_corr1, bias_corr2}: lets a captured CUDA graph see per-step values.
  const float* hyper;
};

// p (fp32 master), m, v updated in place; shadow (bf16 copy used by the forward) rewritten when present.
// update = lr * (m / bc1) / (sqrt(v / bc2) + eps) + lr * wd * p   (decoupled decay), grad pre-multiplied by ctrl[1].
template <typename TG>
__global__ void __launch_bounds__(kOptThreads)
adam_flat_kernel(float* __restrict__ p, __nv_bfloat16* __restrict__ shadow, const TG* __restrict__ g,
                 float* __restrict__ m, float* __restrict__ v, long long n, const float* __restrict__ ctrl,
                 AdamArgs a) {
  if (a.hyper) {
    a.lr = a.hyper[0];
    a.bias_corr1 = a.hyper[1];
    a.bias_corr2 = a.hyper[2];
  }
  const float gscale = ctrl ? ctrl[1] : 1.0f;
  if (ctrl && a.skip_if_nonfinite && ctrl[2] == 0.0f) return;
  const float inv_bc1 = 1.0f / a.bias_corr1, inv_bc2 = 1.0f / a.bias_corr2;
  const long long nv = n / 8 * 8;
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < nv; i += stride) {
    float gv[8], pv[8], mv[8], vv[8];
    Vec8<TG>::load(g + i, gv);
    Vec8<float>::load(p + i, pv);
    Vec8<float>::load(m + i, mv);
    Vec8<float>::load(v + i, vv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gr = gv[j] * gscale;
      mv[j] = a.beta1 * mv[j] + (1.0f - a.beta1) * gr;
      vv[j] = a.beta2 * vv[j] + (1.0f - a.beta2) * gr * gr;
      const float upd = a.lr * (mv[j] * inv_bc1) / (sqrtf(vv[j] * inv_bc2) + a.eps) + a.lr * a.weight_decay * pv[j];
      pv[j] -= upd;
    }
    Vec8<float>::store(p + i, pv);
    Vec8<float>::store(m + i, mv);
    Vec8<float>::store(v + i, vv);
    if (shadow) Vec8<__nv_bfloat16>::store(shadow + i, pv);
  }
  if (blockIdx.x == 0)
    for (long long i = nv + threadIdx.x; i < n; i += blockDim.x) {
      const float gr = to_f32(g[i]) * gscale;
      const float mm = a.beta1 * m[i] + (1.0f - a.beta1) * gr;
      const float vv = a.beta2 * v[i] + (1.0f - a.beta2) * gr * gr;
      const float pp = p[i] - (a.lr * (mm * inv_bc1) / (sqrtf(vv * inv_bc2) + a.eps) + a.lr * a.weight_decay * p[i]);
      m[i] = mm; v[i] = vv; p[i] = pp;
      if (shadow) shadow[i] = __float2bfloat16(pp);
    }
}

// SGD: g += wd * p (L2); buf = first ? g : momentum * buf + g; p -= lr * (momentum ? buf : g)
// (reference: lib/core/optim/sgd.dart:35-83).
template <typename TG>
__global__ void __launch_bounds__(kOptThreads)
sgd_flat_kernel(float* __restrict__ p, __nv_bfloat16* __restrict__ shadow, const TG* __restrict__ g,
                float* __restrict__ buf, long long n, const float* __restrict__ ctrl, float lr, float momentum,
                float weight_decay, int first_step) {
  const float gscale = ctrl ? ctrl[1] : 1.0f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float gr = to_f32(g[i]) * gscale + weight_decay * p[i];
    if (momentum != 0.0f) {
      const float b = first_step ? gr : momentum * buf[i] + gr;
      buf[i] = b;
      gr = b;
    }
    const float pp = p[i] - lr * gr;
    p[i] = pp;
    if (shadow) shadow[i] = __float2bfloat16(pp);
  }
}

static inline int flat_grid(long long n, int per_thread) {
  long long blocks = (n + (long long)kOptThreads * per_thread - 1) / ((long long)kOptThreads * per_thread);
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace dptb

using namespace dptb;

// Number of partial sums dptb_sqnorm writes for a range of n elements (size the scratch with this).
extern "C" int dptb_sqnorm_parts(long long n) { return flat_grid(n, 8); }

// grad dtype: 0 fp32, 1 bf16.  partial: fp32 scratch of dptb_sqnorm_parts(n) floats.  Then finalises ctrl.
extern "C" int dptb_grad_norm(const void* g, long long n, int gdtype, float* partial, float* ctrl, float max_norm,
                              int add_previous, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  const int parts = flat_grid(n, 8);
  if ((reinterpret_cast<uintptr_t>(g) & 31) != 0) return kErrBadShape;
  if (gdtype) sqnorm_partial_kernel<__nv_bfloat16><<<parts, kOptThreads, 0, st>>>((const __nv_bfloat16*)g, n, partial);
  else        sqnorm_partial_kernel<float><<<parts, kOptThreads, 0, st>>>((const float*)g, n, partial);
  DPTB_CUDA_OK(cudaGetLastError());
  clip_finalize_kernel<<<1, 1024, 0, st>>>(partial, parts, ctrl, max_norm, add_previous);
  return counted(2, (int)cudaGetLastError());
}
extern "C" int dptb_scale_by_ctrl(void* g, long long n, int gdtype, const float* ctrl, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  if (gdtype) scale_by_ctrl_kernel<__nv_bfloat16><<<flat_grid(n, 1), kOptThreads, 0, st>>>((__nv_bfloat16*)g, n, ctrl);
  else        scale_by_ctrl_kernel<float><<<flat_grid(n, 1), kOptThreads, 0, st>>>((float*)g, n, ctrl);
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_adam_flat(float* p, void* shadow, const void* g, int gdtype, float* m, float* v, long long n,
                              const float* ctrl, float lr, float beta1, float beta2, float eps, float weight_decay,
                              float bias_corr1, float bias_corr2, int skip_if_nonfinite, const float* hyper,
                              void* stream) {
  if (n <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  if (((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
        reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(shadow)) & 31) != 0)
    return kErrBadShape;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, skip_if_nonfinite, hyper};
  if (gdtype) adam_flat_kernel<__nv_bfloat16><<<flat_grid(n, 8), kOptThreads, 0, st>>>(p, (__nv_bfloat16*)shadow, (const __nv_bfloat16*)g, m, v, n, ctrl, a);
  else        adam_flat_kernel<float><<<flat_grid(n, 8), kOptThreads, 0, st>>>(p, (__nv_bfloat16*)shadow, (const float*)g, m, v, n, ctrl, a);
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_sgd_flat(float* p, void* shadow, const void* g, int gdtype, float* buf, long long n,
                             const float* ctrl, float lr, float momentum, float weight_decay, int first_step,
                             void* stream) {
  if (n <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  if (gdtype) sgd_flat_kernel<__nv_bfloat16><<<flat_grid(n, 1), kOptThreads, 0, st>>>(p, (__nv_bfloat16*)shadow, (const __nv_bfloat16*)g, buf, n, ctrl, lr, momentum, weight_decay, first_step);
  else        sgd_flat_kernel<float><<<flat_grid(n, 1), kOptThreads, 0, st>>>(p, (__nv_bfloat16*)shadow, (const float*)g, buf, n, ctrl, lr, momentum, weight_decay, first_step);
  return counted(1, (int)cudaGetLastError());
}
