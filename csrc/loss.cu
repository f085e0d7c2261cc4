// Row softmax (forward / backward) and fused softmax + cross-entropy over a padded logits buffer.
//
// Cross-entropy never writes probabilities: the forward keeps one log-sum-exp per row, the backward
// rebuilds (softmax - onehot) * upstream in place over the logits buffer.  (A single-pass variant that staged each
// row in shared memory and wrote the gradient during the forward was built and measured: 1.13 ms against 0.41 + 0.59 ms
// for the two passes at 16384 x 50304, because one resident row per SM serialises the two exponential passes; the
// training step did not get faster, so the two kernels stay.)
// (reference: lib/native/src/kernels/softmax.cuh:24-160, lib/core/tensor/softmax.dart:100-212).
#include "common/host.h"
#include "common/reduce.cuh"

namespace dptb {

constexpr int kLossThreads = 256;

// (max, sum of exp(x - max)) pairs combine associatively.
__device__ __forceinline__ void online_combine(float& m, float& s, float m2, float s2) {
  const float nm = fmaxf(m, m2);
  if (nm == -INFINITY) { m = nm; s = 0.0f; return; }
  s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  m = nm;
}

template <typename T>
__device__ __forceinline__ void row_online_max_sum(const T* __restrict__ xr, int V, bool vec_ok, float& m, float& s) {
  m = -INFINITY;
  s = 0.0f;
  if (vec_ok) {
    const int nvec = V / 8;
    for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
      float v[8];
      Vec8<T>::load(xr + vi * 8, v);
      float lm = v[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, v[j]);
      float ls = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ls += __expf(v[j] - lm);
      online_combine(m, s, lm, ls);
    }
    for (int c = nvec * 8 + threadIdx.x; c < V; c += blockDim.x) online_combine(m, s, to_f32(xr[c]), 1.0f);
  } else {
    for (int c = threadIdx.x; c < V; c += blockDim.x) online_combine(m, s, to_f32(xr[c]), 1.0f);
  }
}

// Block-wide combine of (m, s); result broadcast.  scratch: 66 floats.
__device__ __forceinline__ void block_online_combine(float& m, float& s, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_combine(m, s, m2, s2);
  }
  __syncthreads();
  if (lane == 0) { scratch[warp] = m; scratch[32 + warp] = s; }
  __syncthreads();
  if (warp == 0) {
    float mm = lane < nw ? scratch[lane] : -INFINITY;
    float ss = lane < nw ? scratch[32 + lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, mm, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, ss, o);
      online_combine(mm, ss, m2, s2);
    }
    if (lane == 0) { scratch[64] = mm; scratch[65] = ss; }
  }
  __syncthreads();
  m = scratch[64];
  s = scratch[65];
}

// loss[r] = lse(x[r, :V]) - x[r, tgt[r]];  lse saved for the backward.  Targets outside [0, V) give loss = lse
// (no picked logit), matching an all-zero one-hot row.
template <typename T>
__global__ void __launch_bounds__(kLossThreads)
ce_fwd_kernel(const T* __restrict__ logits, long long ld, const long long* __restrict__ targets,
              float* __restrict__ loss, float* __restrict__ lse_out, long long rows, int V, int vec_ok) {
  __shared__ float scratch[66];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = logits + r * ld;
    float m, s;
    row_online_max_sum(xr, V, vec_ok != 0, m, s);
    block_online_combine(m, s, scratch);
    if (threadIdx.x == 0) {
      const float lse = m + logf(s);
      const long long t = targets[r];
      const float picked = (t >= 0 && t < V) ? to_f32(xr[t]) : 0.0f;
      lse_out[r] = lse;
      loss[r] = (t >= 0 && t < V) ? lse - picked : lse;
    }
  }
}

// dlogits[r, c] = (exp(x[r,c] - lse[r]) - [c == tgt[r]]) * g[r * g_stride] * scale for c < V, 0 for V <= c < ld_used.
// May run in place (dlogits == logits).
template <typename T>
__global__ void __launch_bounds__(kLossThreads)
ce_bwd_kernel(const T* logits, long long ld, const long long* __restrict__ targets, const float* __restrict__ lse,
              const float* __restrict__ g, int g_stride, float scale, T* dlogits, long long ldd, long long rows,
              int V, int pad_to, int vec_ok) {
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = logits + r * ld;
    T* dr = dlogits + r * ldd;
    const float l = lse[r];
    const float gs = g[r * g_stride] * scale;
    const long long t = targets[r];
    if (vec_ok) {
      const int nvec = pad_to / 8;
      for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
        float v[8];
        Vec8<T>::load(xr + vi * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = vi * 8 + j;
          float p = c < V ? __expf(v[j] - l) : 0.0f;
          if (c == t) p -= 1.0f;
          v[j] = p * gs;
        }
        Vec8<T>::store(dr + vi * 8, v);
      }
    } else {
      for (int c = threadIdx.x; c < pad_to; c += blockDim.x) {
        float p = c < V ? __expf(to_f32(xr[c]) - l) : 0.0f;
        if (c == t) p -= 1.0f;
        dr[c] = from_f32<T>(p * gs);
      }
    }
  }
}

// y = softmax(x) per row (three passes; rows are L2 resident between passes).
template <typename T>
__global__ void __launch_bounds__(kLossThreads)
softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int D) {
  __shared__ float scratch[66];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * D;
    float m, s;
    row_online_max_sum(xr, D, false, m, s);
    block_online_combine(m, s, scratch);
    const float inv = 1.0f / s;
    for (int c = threadIdx.x; c < D; c += blockDim.x) y[r * D + c] = from_f32<T>(__expf(to_f32(xr[c]) - m) * inv);
  }
}
// dx = (dy - <dy, y>) * y
template <typename T>
__global__ void __launch_bounds__(kLossThreads)
softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, long long rows, int D) {
  __shared__ float scratch[33];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    float dot = 0.0f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) dot += to_f32(y[r * D + c]) * to_f32(dy[r * D + c]);
    dot = block_sum(dot, scratch);
    for (int c = threadIdx.x; c < D; c += blockDim.x)
      dx[r * D + c] = from_f32<T>((to_f32(dy[r * D + c]) - dot) * to_f32(y[r * D + c]));
  }
}

// Deterministic mean of a float vector into out[0] (single CTA; used for the scalar loss).
__global__ void __launch_bounds__(1024) mean_f32_kernel(const float* __restrict__ x, long long n, float* out, float scale) {
  __shared__ float scratch[33];
  float s = 0.0f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) out[0] = s * scale;
}

static inline int row_grid(long long rows) {
  const long long cap = (long long)sm_count() * 16;
  return (int)(rows < cap ? rows : cap);
}

}  // namespace dptb

using namespace dptb;

extern "C" int dptb_ce_fwd(const void* logits, long long ld, const long long* targets, float* loss, float* lse,
                           long long rows, int V, int dtype, void* stream) {
  if (rows <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  const int vec_ok = ((reinterpret_cast<uintptr_t>(logits) & 15) == 0) && (ld % 8 == 0);
  if (dtype) ce_fwd_kernel<__nv_bfloat16><<<row_grid(rows), kLossThreads, 0, st>>>((const __nv_bfloat16*)logits, ld, targets, loss, lse, rows, V, vec_ok);
  else       ce_fwd_kernel<float><<<row_grid(rows), kLossThreads, 0, st>>>((const float*)logits, ld, targets, loss, lse, rows, V, vec_ok);
  return counted(1, (int)cudaGetLastError());
}
// pad_to: number of leading columns of each dlogits row to write (V <= pad_to <= ldd); columns in [V, pad_to) get 0.
extern "C" int dptb_ce_bwd(const void* logits, long long ld, const long long* targets, const float* lse, const float* g,
                           int g_stride, float scale, void* dlogits, long long ldd, long long rows, int V, int pad_to,
                           int dtype, void* stream) {
  if (rows <= 0) return 0;
  if (pad_to < V || pad_to > ldd || pad_to > ld) return kErrBadShape;
  auto st = static_cast<cudaStream_t>(stream);
  const int vec_ok = (((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(dlogits)) & 15) == 0) &&
                     (ld % 8 == 0) && (ldd % 8 == 0) && (pad_to % 8 == 0);
  if (dtype) ce_bwd_kernel<__nv_bfloat16><<<row_grid(rows), kLossThreads, 0, st>>>((const __nv_bfloat16*)logits, ld, targets, lse, g, g_stride, scale, (__nv_bfloat16*)dlogits, ldd, rows, V, pad_to, vec_ok);
  else       ce_bwd_kernel<float><<<row_grid(rows), kLossThreads, 0, st>>>((const float*)logits, ld, targets, lse, g, g_stride, scale, (float*)dlogits, ldd, rows, V, pad_to, vec_ok);
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_softmax_fwd(const void* x, void* y, long long rows, int D, int dtype, void* stream) {
  if (rows <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype) softmax_fwd_kernel<__nv_bfloat16><<<row_grid(rows), kLossThreads, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, D);
  else       softmax_fwd_kernel<float><<<row_grid(rows), kLossThreads, 0, st>>>((const float*)x, (float*)y, rows, D);
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_softmax_bwd(const void* y, const void* dy, void* dx, long long rows, int D, int dtype, void* stream) {
  if (rows <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype) softmax_bwd_kernel<__nv_bfloat16><<<row_grid(rows), kLossThreads, 0, st>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, rows, D);
  else       softmax_bwd_kernel<float><<<row_grid(rows), kLossThreads, 0, st>>>((const float*)y, (const float*)dy, (float*)dx, rows, D);
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_mean_f32(const float* x, long long n, float* out, float scale, void* stream) {
  mean_f32_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(x, n, out, scale);
  return counted(1, (int)cudaGetLastError());
}
