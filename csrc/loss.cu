// Row softmax (forward / backward) and fused softmax + cross-entropy over a padded logits buffer.
//
// Cross-entropy never writes probabilities: the forward keeps one log-sum-exp per row, the backward
// rebuilds (softmax - onehot) * upstream in place over the logits buffer
// (reference: lib/native/src/kernels/softmax.cuh:24-160, lib/core/tensor/softmax.dart:100-212).
#include "common/host.h"
#include "common/ptx.cuh"
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

// Loss and gradient in ONE pass over HBM.  A CTA streams rows of logits through two shared-memory buffers: a producer
// warp brings row i + 1 in with one bulk copy (completion on an mbarrier) while the 16 compute warps fold (max, sum exp)
// over row i, derive its log-sum-exp and loss, overwrite the row in shared memory with (softmax - onehot) * scale, and
// hand it back to the producer, which writes it over the logits with one bulk store.  The logits are read once and
// written once (the two-kernel path reads them twice); the upstream scalar of the mean loss is applied by the caller
// to the small operands of the following GEMMs.  Requires two rows (pad_to elements each) to fit in shared memory.
constexpr int kCeComputeThreads = 512;
constexpr int kCeFusedThreads = kCeComputeThreads + 32;

__device__ __forceinline__ void ce_bar_compute() { asm volatile("bar.sync 1, 512;" ::: "memory"); }
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store_1d(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kCeFusedThreads)
ce_fused_kernel(T* logits, long long ld, const long long* __restrict__ targets, float* __restrict__ loss,
                float* __restrict__ lse_out, float scale, long long rows, int V, int pad_to, int row_bytes) {
  extern __shared__ __align__(128) unsigned char ce_smem[];
  __shared__ uint64_t bars[4];            // full[2] (row landed), done[2] (row rewritten, ready to store)
  __shared__ float scratch[66];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  uint64_t* full = bars;
  uint64_t* done = bars + 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long n_mine = rows > blockIdx.x ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int b = 0; b < 2; ++b) {
      mbar_init(&full[b], 1);
      mbar_init(&done[b], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  const uint32_t bytes = (uint32_t)pad_to * sizeof(T);

  if (warp == kCeComputeThreads / 32) {
    // ------------------------------------------------------------------ producer warp: bulk loads and stores
    if (lane == 0) {
      for (long long i = 0; i < n_mine && i < 2; ++i) {
        mbar_arrive_expect_tx(&full[i], bytes);
        bulk_load_1d(ce_smem + i * row_bytes, logits + (blockIdx.x + i * gridDim.x) * ld, bytes, &full[i]);
      }
      for (long long i = 0; i < n_mine; ++i) {
        const int b = (int)(i & 1);
        if (!mbar_wait(&done[b], (uint32_t)(i >> 1) & 1, abort_flag, kWaitFlagTimeout)) break;
        bulk_store_1d(logits + (blockIdx.x + i * gridDim.x) * ld, ce_smem + b * row_bytes, bytes);
        bulk_commit_group();
        if (i + 2 < n_mine) {
          bulk_wait_read_all();            // the store has read the buffer: it may receive the row after next
          mbar_arrive_expect_tx(&full[b], bytes);
          bulk_load_1d(ce_smem + b * row_bytes, logits + (blockIdx.x + (i + 2) * gridDim.x) * ld, bytes, &full[b]);
        }
      }
      bulk_wait_all();                     // every store has completed before the CTA leaves
    }
    return;
  }
  // -------------------------------------------------------------------- compute warps
  const int nvec_v = V / 8, nvec = pad_to / 8;
  for (long long i = 0; i < n_mine; ++i) {
    const long long r = blockIdx.x + i * gridDim.x;
    const int b = (int)(i & 1);
    T* srow = reinterpret_cast<T*>(ce_smem + b * row_bytes);
    if (!mbar_wait(&full[b], (uint32_t)(i >> 1) & 1, abort_flag, kWaitFullTimeout)) break;
    float m = -INFINITY, s = 0.0f;
    for (int vi = threadIdx.x; vi < nvec_v; vi += kCeComputeThreads) {
      float v[8];
      Vec8<T>::load(srow + vi * 8, v);
      float lm = v[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, v[j]);
      float ls = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ls += __expf(v[j] - lm);
      online_combine(m, s, lm, ls);
    }
    for (int c = nvec_v * 8 + threadIdx.x; c < V; c += kCeComputeThreads) online_combine(m, s, to_f32(srow[c]), 1.0f);
    // combine over the 512 compute threads (named barrier: the producer warp does not take part)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_combine(m, s, m2, s2);
    }
    ce_bar_compute();                      // scratch of the previous row has been read by everyone
    if (lane == 0) { scratch[warp] = m; scratch[32 + warp] = s; }
    ce_bar_compute();
    float mm = lane < kCeComputeThreads / 32 ? scratch[lane] : -INFINITY;
    float ss = lane < kCeComputeThreads / 32 ? scratch[32 + lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, mm, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, ss, o);
      online_combine(mm, ss, m2, s2);
    }
    const float l = mm + logf(ss);
    const long long t = targets[r];
    if (threadIdx.x == 0) {
      const float picked = (t >= 0 && t < V) ? to_f32(srow[t]) : 0.0f;
      lse_out[r] = l;
      loss[r] = (t >= 0 && t < V) ? l - picked : l;
    }
    ce_bar_compute();                      // the picked logit has been read before the row is overwritten
    for (int vi = threadIdx.x; vi < nvec; vi += kCeComputeThreads) {
      float v[8];
      Vec8<T>::load(srow + vi * 8, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = vi * 8 + j;
        float p = c < V ? __expf(v[j] - l) : 0.0f;
        if (c == t) p -= 1.0f;
        v[j] = p * scale;
      }
      Vec8<T>::store(srow + vi * 8, v);
    }
    fence_proxy_async_smem();              // the bulk store reads what these threads wrote
    ce_bar_compute();
    if (threadIdx.x == 0) mbar_arrive(&done[b]);
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
// Fused loss + in-place gradient (see ce_fused_kernel).  Returns kErrUnsupported when two rows do not fit in shared
// memory or the buffer cannot be moved by 16-byte bulk copies: the caller then runs dptb_ce_fwd + dptb_ce_bwd.
extern "C" int dptb_ce_fused(void* logits, long long ld, const long long* targets, float* loss, float* lse, float scale,
                             long long rows, int V, int pad_to, int dtype, void* stream) {
  if (rows <= 0) return 0;
  if (pad_to < V || pad_to > ld) return kErrBadShape;
  const size_t esz = dtype ? 2 : 4;
  const size_t row_bytes = ((size_t)pad_to * esz + 127) / 128 * 128;
  if ((reinterpret_cast<uintptr_t>(logits) & 15) || (ld % 8) || (pad_to % 8) || 2 * row_bytes > 220 * 1024) return kErrUnsupported;
  auto st = static_cast<cudaStream_t>(stream);
  const int per_sm = 4 * row_bytes <= 220 * 1024 ? 2 : 1;
  const long long want = (long long)sm_count() * per_sm;
  const int grid = (int)(rows < want ? rows : want);
  const size_t smem = 2 * row_bytes;
  if (dtype) {
    auto kern = ce_fused_kernel<__nv_bfloat16>;
    DPTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kCeFusedThreads, smem, st>>>((__nv_bfloat16*)logits, ld, targets, loss, lse, scale, rows, V, pad_to, (int)row_bytes);
  } else {
    auto kern = ce_fused_kernel<float>;
    DPTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kCeFusedThreads, smem, st>>>((float*)logits, ld, targets, loss, lse, scale, rows, V, pad_to, (int)row_bytes);
  }
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
