// LayerNorm and RMSNorm, forward and backward, for bf16 or fp32 rows.
//
// Forward: one pass over each row held in registers (16-byte vector loads), centred variance.
// Backward: dX per row in the same pass as per-column partial sums of dGamma / dBeta, which are
// reduced in two deterministic stages (per-CTA partials in scratch, then a column reduce) instead
// of the reference's one-atomicAdd-per-element scheme
// (reference: lib/native/src/kernels/layernorm.cuh:22-122, lib/native/src/kernels/rms_norm.cuh:20-96).
#include "common/host.h"
#include "common/reduce.cuh"

namespace dptb {

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // 8-element vectors per thread held in registers (template parameter V <= this)

template <int G>
__device__ __forceinline__ float group_sum(float v, float* scratch) {
  if (G == 32) return warp_sum(v);
  return block_sum(v, scratch);
}

// G threads cooperate on one row; a block of 256 threads handles 256 / G rows per iteration.
template <typename T, int G, int V, bool RMS>
__global__ void __launch_bounds__(kNormThreads, 3)
norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, long long rows, int D, float eps) {
  __shared__ float scratch[33];
  pdl_wait();                // (programmatic dependent launch: no-ops in an ordinary launch)
  pdl_launch_dependents();
  constexpr int RPB = kNormThreads / G;
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const int nvec = D / 8;
  for (long long base = (long long)blockIdx.x * RPB; base < rows; base += (long long)gridDim.x * RPB) {
    const long long r = base + g;
    const bool live = r < rows;
    float v[V][8];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int vi = t + i * G;
      if (live && vi < nvec) {
        Vec8<T>::load(x + r * D + vi * 8, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += RMS ? v[i][j] * v[i][j] : v[i][j];
      }
    }
    s = group_sum<G>(s, scratch);
    float mean = 0.0f, rstd;
    if (RMS) {
      rstd = rsqrtf(s / D + eps);
    } else {
      mean = s / D;
      float q = 0.0f;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const int vi = t + i * G;
        if (live && vi < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float d = v[i][j] - mean;
            q += d * d;
          }
        }
      }
      q = group_sum<G>(q, scratch);
      rstd = rsqrtf(q / D + eps);
    }
    if (live && t == 0) {
      if (mean_out) mean_out[r] = mean;
      if (rstd_out) rstd_out[r] = rstd;
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int vi = t + i * G;
      if (live && vi < nvec) {
        float gm[8], bt[8], o[8];
        Vec8<T>::load(gamma + vi * 8, gm);
        if (!RMS && beta) Vec8<T>::load(beta + vi * 8, bt);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = (v[i][j] - mean) * rstd * gm[j];
          if (!RMS && beta) o[j] += bt[j];
        }
        Vec8<T>::store(y + r * D + vi * 8, o);
      }
    }
  }
}

// Any D (no alignment requirement): one CTA per row, three passes from global memory.
template <typename T, bool RMS>
__global__ void __launch_bounds__(kNormThreads)
norm_fwd_generic_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                        T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, long long rows,
                        int D, float eps) {
  __shared__ float scratch[33];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * D;
    float s = 0.0f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      const float a = to_f32(xr[c]);
      s += RMS ? a * a : a;
    }
    s = block_sum(s, scratch);
    float mean = 0.0f, rstd;
    if (RMS) {
      rstd = rsqrtf(s / D + eps);
    } else {
      mean = s / D;
      float q = 0.0f;
      for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float d = to_f32(xr[c]) - mean;
        q += d * d;
      }
      q = block_sum(q, scratch);
      rstd = rsqrtf(q / D + eps);
    }
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[r] = mean;
      if (rstd_out) rstd_out[r] = rstd;
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      float o = (to_f32(xr[c]) - mean) * rstd * to_f32(gamma[c]);
      if (!RMS && beta) o += to_f32(beta[c]);
      y[r * D + c] = from_f32<T>(o);
    }
  }
}

// Backward.  partial: [gridDim.x, 2, D] fp32 (dGamma partials then dBeta partials; RMS uses only the first).
// (A third set of partials, the column sums of the dX rows written here, which are the bias gradient of the Linear
// before the norm, was tried so that those Linears need no column-sum pass: the extra 24 accumulators spilled at the
// 128-register budget of two CTAs per SM, 62.5 us against 46.1 + 19.5 + 5.8 us for the separate kernels at
// 16384 x 768, and the training step got 1.5 % slower.  Not kept.)
template <typename T, int G, int V, bool RMS>
__global__ void __launch_bounds__(kNormThreads, 2)
norm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ gamma,
                const float* __restrict__ mean_in, const float* __restrict__ rstd_in, const T* __restrict__ dres,
                T* __restrict__ dx, float* __restrict__ partial, long long rows, int D) {
  extern __shared__ float red[];  // [RPB][D] when RPB > 1
  __shared__ float scratch[33];
  constexpr int RPB = kNormThreads / G;
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const int nvec = D / 8;
  float dg_acc[V][8], db_acc[V][8];
#pragma unroll
  for (int i = 0; i < V; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dg_acc[i][j] = db_acc[i][j] = 0.0f;

  for (long long base = (long long)blockIdx.x * RPB; base < rows; base += (long long)gridDim.x * RPB) {
    const long long r = base + g;
    const bool live = r < rows;
    const float mean = (live && !RMS) ? mean_in[r] : 0.0f;
    const float rstd = live ? rstd_in[r] : 0.0f;
    // All loads of the row are issued up front and kept packed; values are unpacked (and x-hat recomputed) in both
    // passes, which costs a few FMAs and saves the registers that would cap occupancy.
    Raw8<T> xr[V], dr[V], rr[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int vi = t + i * G;
      if (live && vi < nvec) {
        xr[i].load(x + r * D + vi * 8);
        dr[i].load(dy + r * D + vi * 8);
        if (dres) rr[i].load(dres + r * D + vi * 8);
      }
    }
    float c1 = 0.0f, c2 = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int vi = t + i * G;
      if (live && vi < nvec) {
        float xv[8], dv[8], gm[8];
        xr[i].unpack(xv);
        dr[i].unpack(dv);
        Vec8<T>::load(gamma + vi * 8, gm);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          const float gy = dv[j] * gm[j];
          dg_acc[i][j] += dv[j] * xh;
          db_acc[i][j] += dv[j];
          c1 += gy;
          c2 += gy * xh;
        }
      }
    }
    if (!RMS) c1 = group_sum<G>(c1, scratch) / D;
    c2 = group_sum<G>(c2, scratch) / D;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int vi = t + i * G;
      if (live && vi < nvec) {
        float xv[8], dv[8], gm[8], o[8];
        xr[i].unpack(xv);
        dr[i].unpack(dv);
        Vec8<T>::load(gamma + vi * 8, gm);
        if (dres) rr[i].unpack(o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          const float gy = dv[j] * gm[j];
          const float d = RMS ? rstd * (gy - xh * c2) : rstd * (gy - c1 - xh * c2);
          o[j] = dres ? o[j] + d : d;
        }
        Vec8<T>::store(dx + r * D + vi * 8, o);
      }
    }
  }

  // Stage 1 of the parameter-gradient reduction: fold the row groups of this CTA, fixed order.
  float* pg = partial + (long long)blockIdx.x * 2 * D;
  for (int pass = 0; pass < (RMS ? 1 : 2); ++pass) {
    if (RPB > 1) {
      __syncthreads();
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const int vi = t + i * G;
        if (vi < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) red[g * D + vi * 8 + j] = pass == 0 ? dg_acc[i][j] : db_acc[i][j];
        }
      }
      __syncthreads();
      for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < RPB; ++k) s += red[k * D + c];
        pg[pass * D + c] = s;
      }
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const int vi = t + i * G;
        if (vi < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) pg[pass * D + vi * 8 + j] = pass == 0 ? dg_acc[i][j] : db_acc[i][j];
        }
      }
    }
  }
}

// Stage 2: out[c] (+)= sum_b partial[b, which, c].  32 columns x 8 slices of the partial rows per CTA.
template <typename T>
__global__ void __launch_bounds__(256)
norm_param_grad_reduce_kernel(const float* __restrict__ partial, int nparts, int D, T* __restrict__ dgamma,
                              T* __restrict__ dbeta, int accumulate) {
  __shared__ float sm[8][33];
  const int cx = threadIdx.x & 31, sl = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  for (int which = 0; which < 2; ++which) {
    T* out = which == 0 ? dgamma : dbeta;
    if (!out) continue;  // uniform
    float s = 0.0f;
    if (c < D)
      for (int b = sl; b < nparts; b += 8) s += partial[((long long)b * 2 + which) * D + c];
    __syncthreads();
    sm[sl][cx] = s;
    __syncthreads();
    if (sl == 0 && c < D) {
      float tot = 0.0f;
#pragma unroll
      for (int k = 0; k < 8; ++k) tot += sm[k][cx];
      if (accumulate) tot += to_f32(out[c]);
      out[c] = from_f32<T>(tot);
    }
  }
}

// Generic backward for any D: one CTA per row for dX, atomics-free column pass for the parameter gradients
// is replaced by per-CTA partials as above (each CTA strides over rows and owns all columns).
template <typename T, bool RMS>
__global__ void __launch_bounds__(kNormThreads)
norm_bwd_generic_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ gamma,
                        const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                        const T* __restrict__ dres, T* __restrict__ dx, float* __restrict__ partial, long long rows,
                        int D) {
  __shared__ float scratch[33];
  float* pg = partial + (long long)blockIdx.x * 2 * D;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    pg[c] = 0.0f;
    pg[D + c] = 0.0f;
  }
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float mean = RMS ? 0.0f : mean_in[r];
    const float rstd = rstd_in[r];
    float c1 = 0.0f, c2 = 0.0f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      const float xh = (to_f32(x[r * D + c]) - mean) * rstd;
      const float gy = to_f32(dy[r * D + c]) * to_f32(gamma[c]);
      c1 += gy;
      c2 += gy * xh;
    }
    c1 = RMS ? 0.0f : block_sum(c1, scratch) / D;
    c2 = block_sum(c2, scratch) / D;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      const float xh = (to_f32(x[r * D + c]) - mean) * rstd;
      const float d = to_f32(dy[r * D + c]);
      const float gy = d * to_f32(gamma[c]);
      float o = rstd * (gy - c1 - xh * c2);
      if (dres) o += to_f32(dres[r * D + c]);
      dx[r * D + c] = from_f32<T>(o);
      pg[c] += d * xh;  // each thread owns its columns: no race, fixed order
      pg[D + c] += d;
    }
  }
}

// Pick (G, V): 32 threads per row while a row fits 4 vectors per lane (D <= 1024), else the whole CTA per row.
#define DPTB_NORM_DISPATCH_V(V_, ...) \
  switch (V_) {                        \
    case 1: { constexpr int V = 1; __VA_ARGS__; } break; \
    case 2: { constexpr int V = 2; __VA_ARGS__; } break; \
    case 3: { constexpr int V = 3; __VA_ARGS__; } break; \
    default: { constexpr int V = 4; __VA_ARGS__; } break; \
  }

template <typename T, bool RMS>
static int norm_fwd_launch(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                           long long rows, int D, float eps, cudaStream_t st) {
  if (rows <= 0) return 0;
  const bool al = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                    reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta)) & 15) == 0;
  const int nsm = sm_count();
  const int nvec = D / 8;
  if (al && D % 8 == 0 && nvec <= 32 * kNormMaxVec) {
    long long blocks = (rows + 7) / 8;
    if (blocks > nsm * 8) blocks = nsm * 8;
    DPTB_NORM_DISPATCH_V((nvec + 31) / 32, (launch_k(norm_fwd_kernel<T, 32, V, RMS>, dim3((int)blocks), dim3(kNormThreads), 0, st,
                 (const T*)x, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, D, eps)));
  } else if (al && D % 8 == 0 && nvec <= 256 * kNormMaxVec) {
    long long blocks = rows < nsm * 8 ? rows : nsm * 8;
    DPTB_NORM_DISPATCH_V((nvec + 255) / 256, (launch_k(norm_fwd_kernel<T, 256, V, RMS>, dim3((int)blocks), dim3(kNormThreads), 0, st,
                 (const T*)x, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, D, eps)));
  } else {
    long long blocks = rows < nsm * 8 ? rows : nsm * 8;
    norm_fwd_generic_kernel<T, RMS><<<(int)blocks, kNormThreads, 0, st>>>((const T*)x, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, D, eps);
  }
  return counted(1, (int)cudaGetLastError());
}

template <typename T, bool RMS>
static int norm_bwd_launch(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd,
                           const void* dres, void* dx, void* dgamma, void* dbeta, float* partial, int partial_rows,
                           int accumulate, long long rows, int D, cudaStream_t st, int stage1_only, int* nparts_out) {
  if (rows <= 0) return 0;
  const bool al = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx) |
                    reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(dres)) & 15) == 0;
  int blocks = partial_rows;
  if (blocks <= 0) return kErrBadShape;
  const int nvec = D / 8;
  if (al && D % 8 == 0 && nvec <= 32 * kNormMaxVec) {
    long long need = (rows + 7) / 8;
    if (need < blocks) blocks = (int)need;
    const size_t smem = (size_t)8 * D * sizeof(float);
    DPTB_NORM_DISPATCH_V((nvec + 31) / 32, {
      auto kern = norm_bwd_kernel<T, 32, V, RMS>;
      DPTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 1024 * 4));
      kern<<<blocks, kNormThreads, smem, st>>>((const T*)x, (const T*)dy, (const T*)gamma, mean, rstd, (const T*)dres, (T*)dx, partial, rows, D);
    });
  } else if (al && D % 8 == 0 && nvec <= 256 * kNormMaxVec) {
    if (rows < blocks) blocks = (int)rows;
    DPTB_NORM_DISPATCH_V((nvec + 255) / 256, (norm_bwd_kernel<T, 256, V, RMS><<<blocks, kNormThreads, 0, st>>>(
        (const T*)x, (const T*)dy, (const T*)gamma, mean, rstd, (const T*)dres, (T*)dx, partial, rows, D)));
  } else {
    if (rows < blocks) blocks = (int)rows;
    norm_bwd_generic_kernel<T, RMS><<<blocks, kNormThreads, 0, st>>>((const T*)x, (const T*)dy, (const T*)gamma, mean, rstd, (const T*)dres, (T*)dx, partial, rows, D);
  }
  DPTB_CUDA_OK(cudaGetLastError());
  if (nparts_out) *nparts_out = blocks;
  if (stage1_only) return counted(1, 0);   // the caller runs the parameter-gradient reduction itself (another stream)
  norm_param_grad_reduce_kernel<T><<<(D + 31) / 32, 256, 0, st>>>(partial, blocks, D, (T*)dgamma, RMS ? (T*)nullptr : (T*)dbeta, accumulate);
  return counted(2, (int)cudaGetLastError());
}

}  // namespace dptb

using namespace dptb;

// dtype: 0 = fp32, 1 = bf16 (x, y, gamma, beta share it).  mean / rstd: fp32 [rows] (mean unused for RMS).
extern "C" int dptb_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                                  long long rows, int D, float eps, int dtype, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  return dtype ? norm_fwd_launch<__nv_bfloat16, false>(x, gamma, beta, y, mean, rstd, rows, D, eps, st)
               : norm_fwd_launch<float, false>(x, gamma, beta, y, mean, rstd, rows, D, eps, st);
}
extern "C" int dptb_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, long long rows, int D, float eps,
                                int dtype, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  return dtype ? norm_fwd_launch<__nv_bfloat16, true>(x, gamma, nullptr, y, nullptr, rstd, rows, D, eps, st)
               : norm_fwd_launch<float, true>(x, gamma, nullptr, y, nullptr, rstd, rows, D, eps, st);
}
// partial: fp32 scratch of partial_rows * 2 * D floats.  dres (optional) is added to dx (residual-stream gradient).
// stage1_only: stop after the kernel that writes dx and the per-CTA partials; *nparts_out receives the number of
// partial rows it wrote, and dptb_norm_param_grad_reduce finishes dgamma / dbeta later (on any stream that is ordered
// after this launch).
extern "C" int dptb_layernorm_bwd(const void* x, const void* dy, const void* gamma, const float* mean,
                                  const float* rstd, const void* dres, void* dx, void* dgamma, void* dbeta,
                                  float* partial, int partial_rows, int accumulate, long long rows, int D, int dtype,
                                  void* stream, int stage1_only, int* nparts_out) {
  auto st = static_cast<cudaStream_t>(stream);
  return dtype ? norm_bwd_launch<__nv_bfloat16, false>(x, dy, gamma, mean, rstd, dres, dx, dgamma, dbeta, partial, partial_rows, accumulate, rows, D, st, stage1_only, nparts_out)
               : norm_bwd_launch<float, false>(x, dy, gamma, mean, rstd, dres, dx, dgamma, dbeta, partial, partial_rows, accumulate, rows, D, st, stage1_only, nparts_out);
}
extern "C" int dptb_rmsnorm_bwd(const void* x, const void* dy, const void* gamma, const float* rstd, const void* dres,
                                void* dx, void* dgamma, float* partial, int partial_rows, int accumulate,
                                long long rows, int D, int dtype, void* stream, int stage1_only, int* nparts_out) {
  auto st = static_cast<cudaStream_t>(stream);
  return dtype ? norm_bwd_launch<__nv_bfloat16, true>(x, dy, gamma, nullptr, rstd, dres, dx, dgamma, nullptr, partial, partial_rows, accumulate, rows, D, st, stage1_only, nparts_out)
               : norm_bwd_launch<float, true>(x, dy, gamma, nullptr, rstd, dres, dx, dgamma, nullptr, partial, partial_rows, accumulate, rows, D, st, stage1_only, nparts_out);
}
// Second stage on its own: dgamma (and dbeta, unless null) (+)= column sums of the nparts partial rows.
extern "C" int dptb_norm_param_grad_reduce(const float* partial, int nparts, int D, void* dgamma, void* dbeta,
                                           int accumulate, int dtype, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  if (nparts <= 0 || D <= 0) return 0;
  if (dtype)
    norm_param_grad_reduce_kernel<__nv_bfloat16><<<(D + 31) / 32, 256, 0, st>>>(partial, nparts, D, (__nv_bfloat16*)dgamma, (__nv_bfloat16*)dbeta, accumulate);
  else
    norm_param_grad_reduce_kernel<float><<<(D + 31) / 32, 256, 0, st>>>(partial, nparts, D, (float*)dgamma, (float*)dbeta, accumulate);
  return counted(1, (int)cudaGetLastError());
}
