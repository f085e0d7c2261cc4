// Elementwise, broadcast, reduction, transpose, RoPE, dropout, SwiGLU and sampling kernels.
//
// These keep the tensor-level API of the reference on the device (reference: lib/native/src/kernels/elementwise.cuh,
// lib/native/src/kernels/transpose.cuh, lib/native/src/kernels/matmul.cuh:146-185, lib/native/src/engine.cu:65-88,575-596)
// with its numerical conventions: sign-preserving clamped division, NaN-free pow, log with an optional epsilon.
// Reductions are two-stage and ordered, not one atomicAdd per element.
#include <initializer_list>
#include "common/host.h"
#include "common/reduce.cuh"

namespace dptb {

constexpr int kEwThreads = 256;

static inline int ew_grid(long long n, int per_thread = 1) {
  long long blocks = (n + (long long)kEwThreads * per_thread - 1) / ((long long)kEwThreads * per_thread);
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

__device__ __forceinline__ float safe_recip_mul(float a, float b) {
  const float mag = fmaxf(fabsf(b), 1e-20f);
  return a / (b < 0.0f ? -mag : mag);
}
__device__ __forceinline__ float int_pow(float x, int n) {
  bool neg = n < 0;
  unsigned e = neg ? (unsigned)(-n) : (unsigned)n;
  float r = 1.0f, b = x;
  while (e) {
    if (e & 1u) r *= b;
    b *= b;
    e >>= 1;
  }
  if (!neg) return r;
  return r == 0.0f ? 0.0f : 1.0f / r;
}
__device__ __forceinline__ float safe_pow(float x, float e) {
  const float re = rintf(e);
  if (fabsf(e - re) < 1e-6f) return int_pow(x, (int)re);
  return x > 0.0f ? powf(x, e) : 0.0f;
}

// op: 0 add, 1 sub, 2 mul, 3 div (clamped).  bmode: 0 same shape, 1 b is one element, 2 b is a row of length `cols`
// broadcast over rows, 3 a is one element (scalar on the left).
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
binary_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, long long n, long long cols, int op,
              int bmode) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float x = to_f32(bmode == 3 ? a[0] : a[i]);
    const float y = to_f32(bmode == 0 || bmode == 3 ? b[i] : (bmode == 1 ? b[0] : b[i % cols]));
    float r;
    switch (op) {
      case 0: r = x + y; break;
      case 1: r = x - y; break;
      case 2: r = x * y; break;
      default: r = safe_recip_mul(x, y); break;
    }
    out[i] = from_f32<T>(r);
  }
}

// op: 0 relu 1 sigmoid 2 tanh 3 abs 4 log(x + param) 5 pow(x, param) 6 gelu_tanh 7 quick_gelu 8 silu 9 scale (x*param)
// 10 exp 11 neg 12 sqrt 13 add scalar (x + param)
__device__ __forceinline__ float unary_apply(int op, float x, float param) {
  switch (op) {
    case 0: return fmaxf(x, 0.0f);
    case 1: return 1.0f / (1.0f + expf(-x));
    case 2: return tanhf(x);
    case 3: return fabsf(x);
    case 4: return logf(x + param);
    case 5: return safe_pow(x, param);
    case 6: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + tanhf(u));
    }
    case 7: return x / (1.0f + expf(-1.702f * x));
    case 8: return x / (1.0f + expf(-x));
    case 9: return x * param;
    case 10: return expf(x);
    case 11: return -x;
    case 12: return sqrtf(x);
    case 13: return x + param;
    default: return x;
  }
}
// d(op)/dx evaluated at the forward input x.
__device__ __forceinline__ float unary_grad(int op, float x, float param) {
  switch (op) {
    case 0: return x > 0.0f ? 1.0f : 0.0f;
    case 1: { const float s = 1.0f / (1.0f + expf(-x)); return s * (1.0f - s); }
    case 2: { const float t = tanhf(x); return 1.0f - t * t; }
    case 3: return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : 0.0f);
    case 4: return 1.0f / (x + param);
    case 5: return param * safe_pow(x, param - 1.0f);
    case 6: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      const float t = tanhf(u);
      return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x * x);
    }
    case 7: { const float s = 1.0f / (1.0f + expf(-1.702f * x)); return s + 1.702f * x * s * (1.0f - s); }
    case 8: { const float s = 1.0f / (1.0f + expf(-x)); return s * (1.0f + x * (1.0f - s)); }
    case 9: return param;
    case 10: return expf(x);
    case 11: return -1.0f;
    case 12: return 0.5f / sqrtf(x);
    case 13: return 1.0f;
    default: return 1.0f;
  }
}
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
unary_kernel(const T* __restrict__ x, T* __restrict__ out, long long n, int op, float param) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(unary_apply(op, to_f32(x[i]), param));
}
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
unary_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx, long long n, int op, float param) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dx[i] = from_f32<T>(to_f32(dy[i]) * unary_grad(op, to_f32(x[i]), param));
}

// Column sums of a [rows, cols] matrix with leading dimension ld: stage 1 writes [gridDim.y, cols] partials.
// A block covers 64 columns (32 lanes x 2 adjacent columns) x 8 row lanes; gridDim.x tiles columns, gridDim.y rows.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const T* __restrict__ x, long long ld, long long rows, int cols, float* __restrict__ partial) {
  __shared__ float sm[8][65];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 64 + cx * 2;
  float s0 = 0.0f, s1 = 0.0f;
  const bool pair_ok = (c + 1 < cols) && ((ld & 1) == 0) && ((reinterpret_cast<uintptr_t>(x) & 3) == 0 || sizeof(T) == 4);
  if (c < cols) {
    const long long step = (long long)gridDim.y * 8;
#pragma unroll 4
    for (long long r = (long long)blockIdx.y * 8 + ry; r < rows; r += step) {
      if (pair_ok && sizeof(T) == 2) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(
            reinterpret_cast<const __nv_bfloat16*>(x) + r * ld + c));
        s0 += v.x;
        s1 += v.y;
      } else {
        s0 += to_f32(x[r * ld + c]);
        if (c + 1 < cols) s1 += to_f32(x[r * ld + c + 1]);
      }
    }
  }
  sm[ry][cx * 2] = s0;
  sm[ry][cx * 2 + 1] = s1;
  __syncthreads();
  if (threadIdx.x < 64) {
    const int cc = blockIdx.x * 64 + threadIdx.x;
    if (cc < cols) {
      float t = 0.0f;
#pragma unroll
      for (int k = 0; k < 8; ++k) t += sm[k][threadIdx.x];
      partial[(long long)blockIdx.y * cols + cc] = t;
    }
  }
}
// 16-byte variant for bf16 with cols and ld multiples of 8: a warp covers 256 columns of one row per load, the 8 warps
// of the block take rows round-robin, 4 loads in flight per thread.
__global__ void __launch_bounds__(256)
colsum_partial_vec8_kernel(const __nv_bfloat16* __restrict__ x, long long ld, long long rows, int cols,
                           float* __restrict__ partial) {
  __shared__ float sm[8][257];
  const int lane = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 256 + lane * 8;
  float s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = 0.0f;
  if (c < cols) {
    const long long step = (long long)gridDim.y * 8;
    long long r = (long long)blockIdx.y * 8 + ry;
    for (; r + 3 * step < rows; r += 4 * step) {
      Raw8<__nv_bfloat16> v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u].load(x + (r + u * step) * ld + c);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float f[8];
        v[u].unpack(f);
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j] += f[j];
      }
    }
    for (; r < rows; r += step) {
      float f[8];
      Vec8<__nv_bfloat16>::load(x + r * ld + c, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] += f[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[ry][lane * 8 + j] = s[j];
  __syncthreads();
  const int cc = blockIdx.x * 256 + threadIdx.x;
  if (cc < cols) {
    float t = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sm[k][threadIdx.x];
    partial[(long long)blockIdx.y * cols + cc] = t;
  }
}
// Stage 2 for many partials (a single-launch form in which the last row slice of a column block folded the partials
// was measured slower, 24.6 us against 19.4 us at 16384 x 768: one CTA folding ~200 partials is a serial tail, while this
// kernel spreads the fold over cols / 32 CTAs): a block owns 32 columns, its 8 warps take partials round-robin, fixed-order fold.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_final_wide_kernel(const float* __restrict__ partial, int nparts, int cols, T* __restrict__ out, int accumulate) {
  __shared__ float sm[8][33];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.0f;
  if (c < cols) {
#pragma unroll 4
    for (int p = w; p < nparts; p += 8) s += partial[(long long)p * cols + c];
  }
  sm[w][lane] = s;
  __syncthreads();
  if (w == 0 && c < cols) {
    float t = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sm[k][lane];
    if (accumulate) t += to_f32(out[c]);
    out[c] = from_f32<T>(t);
  }
}
template <typename T>
__global__ void __launch_bounds__(256)
colsum_final_kernel(const float* __restrict__ partial, int nparts, int cols, T* __restrict__ out, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.0f;
#pragma unroll 8
  for (int p = 0; p < nparts; ++p) s += partial[(long long)p * cols + c];
  if (accumulate) s += to_f32(out[c]);
  out[c] = from_f32<T>(s);
}

// Sum of all elements: per-CTA partials, then one CTA folds them in order.  out is fp32[1] scaled by `scale`.
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
sum_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float scratch[33];
  float s = 0.0f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    s += to_f32(x[i]);
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void __launch_bounds__(1024)
sum_final_kernel(const float* __restrict__ partial, int nparts, float* __restrict__ out, float scale) {
  __shared__ float scratch[33];
  float s = 0.0f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) out[0] = s * scale;
}

// out[c, r] = in[r, c]; 32x33 padded tile.
template <typename T>
__global__ void __launch_bounds__(256)
transpose_kernel(const T* __restrict__ in, T* __restrict__ out, long long rows, long long cols) {
  __shared__ T tile[32][33];
  const long long c0 = (long long)blockIdx.x * 32, r0 = (long long)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int k = ty; k < 32; k += 8)
    if (r0 + k < rows && c0 + tx < cols) tile[k][tx] = in[(r0 + k) * cols + c0 + tx];
  __syncthreads();
  for (int k = ty; k < 32; k += 8)
    if (c0 + k < cols && r0 + tx < rows) out[(c0 + k) * rows + r0 + tx] = tile[tx][k];
}

// Strided 2-D copy (slice / concat / pad building block): dst[r*ldd + c] = src[r*lds + c].
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
copy2d_kernel(const T* __restrict__ src, long long lds, T* __restrict__ dst, long long ldd, long long rows, long long cols) {
  const long long n = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols, c = i % cols;
    dst[r * ldd + c] = src[r * lds + c];
  }
}

// Half-split rotary embedding on rows laid out [tokens, heads, head_dim] inside a matrix with row stride `ld`:
// element (t, h, d) sits at x[t*ld + h*head_dim + d].  Position of token t is pos_start + (t % seq_len), or
// positions[t] when given.  `inverse` applies the transpose rotation (the backward).
// inv_freq_i = base^(-2i/rotary_dim); dims >= rotary_dim pass through (reference: lib/core/nn/rotary.dart:95-201).
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
rope_kernel(const T* __restrict__ x, T* __restrict__ out, long long tokens, int heads, int head_dim, int rotary_dim,
            int seq_len, int pos_start, float base, int inverse, const long long* __restrict__ positions,
            long long ld_in, long long ld_out) {
  const int half = rotary_dim / 2;
  const long long per_tok = (long long)heads * half;
  const long long n = tokens * per_tok;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / per_tok;
    const int rem = (int)(i % per_tok);
    const int h = rem / half, d = rem % half;
    const float pos = positions ? (float)positions[t] : (float)(pos_start + (seq_len > 0 ? t % seq_len : t));
    const float inv = powf(base, -2.0f * (float)d / (float)rotary_dim);
    float sn, cs;
    sincosf(pos * inv, &sn, &cs);
    if (inverse) sn = -sn;
    const long long oi = t * ld_in + (long long)h * head_dim + d;
    const long long oo = t * ld_out + (long long)h * head_dim + d;
    const float a = to_f32(x[oi]), b = to_f32(x[oi + half]);
    out[oo] = from_f32<T>(a * cs - b * sn);
    out[oo + half] = from_f32<T>(b * cs + a * sn);
  }
}
// Pass-through copy of the non-rotated tail dims when out != x.
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
rope_tail_kernel(const T* __restrict__ x, T* __restrict__ out, long long tokens, int heads, int head_dim, int rotary_dim,
                 long long ld_in, long long ld_out) {
  const int tail = head_dim - rotary_dim;
  const long long per_tok = (long long)heads * tail;
  const long long n = tokens * per_tok;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / per_tok;
    const int rem = (int)(i % per_tok);
    const int h = rem / tail, d = rotary_dim + rem % tail;
    out[t * ld_out + (long long)h * head_dim + d] = x[t * ld_in + (long long)h * head_dim + d];
  }
}

// Counter-based uniform in [0,1): a keyed 64-bit mix of (seed, offset + index).  The same (seed, offset) reproduces
// the mask, so the backward regenerates it instead of storing it.
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long idx) {
  unsigned long long z = idx + seed * 0x9E3779B97F4A7C15ull + 0x632BE59BD9B4E019ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
dropout_kernel(const T* __restrict__ x, T* __restrict__ out, long long n, float p, unsigned long long seed,
               unsigned long long offset) {
  const float keep_scale = 1.0f / (1.0f - p);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(uniform01(seed, offset + (unsigned long long)i) >= p ? to_f32(x[i]) * keep_scale : 0.0f);
}

// SwiGLU gate: out = silu(g) * u, rows x cols with independent leading dimensions.
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
swiglu_fwd_kernel(const T* __restrict__ g, long long ldg, const T* __restrict__ u, long long ldu, T* __restrict__ out,
                  long long ldo, long long rows, int cols) {
  const long long n = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols;
    const int c = (int)(i % cols);
    const float gv = to_f32(g[r * ldg + c]), uv = to_f32(u[r * ldu + c]);
    out[r * ldo + c] = from_f32<T>(gv / (1.0f + __expf(-gv)) * uv);
  }
}
// 16-byte variants (cols and every leading dimension multiples of 8 elements, 16-byte aligned bases).
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
swiglu_fwd_vec8_kernel(const T* __restrict__ g, long long ldg, const T* __restrict__ u, long long ldu,
                       T* __restrict__ out, long long ldo, long long rows, int cols) {
  pdl_wait();                // (programmatic dependent launch: no-ops in an ordinary launch)
  pdl_launch_dependents();
  const int cv = cols >> 3;
  const long long n = rows * cv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cv;
    const int c = (int)(i - r * cv) << 3;
    float gv[8], uv[8], o[8];
    Vec8<T>::load(g + r * ldg + c, gv);
    Vec8<T>::load(u + r * ldu + c, uv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = gv[j] / (1.0f + __expf(-gv[j])) * uv[j];
    Vec8<T>::store(out + r * ldo + c, o);
  }
}
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
swiglu_bwd_vec8_kernel(const T* __restrict__ g, long long ldg, const T* __restrict__ u, long long ldu,
                       const T* __restrict__ dout, long long ldo, T* __restrict__ dg, long long lddg,
                       T* __restrict__ du, long long lddu, long long rows, int cols) {
  const int cv = cols >> 3;
  const long long n = rows * cv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cv;
    const int c = (int)(i - r * cv) << 3;
    float gv[8], uv[8], d[8], a[8], b[8];
    Vec8<T>::load(g + r * ldg + c, gv);
    Vec8<T>::load(u + r * ldu + c, uv);
    Vec8<T>::load(dout + r * ldo + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.0f / (1.0f + __expf(-gv[j]));
      a[j] = d[j] * uv[j] * sg * (1.0f + gv[j] * (1.0f - sg));
      b[j] = d[j] * gv[j] * sg;
    }
    Vec8<T>::store(dg + r * lddg + c, a);
    Vec8<T>::store(du + r * lddu + c, b);
  }
}
static inline bool vec8_ok(int cols, std::initializer_list<long long> lds, std::initializer_list<const void*> ptrs,
                           int elem_bytes) {
  if (cols & 7) return false;
  for (long long ld : lds) if (ld & 7) return false;
  for (const void* p : ptrs) if (reinterpret_cast<uintptr_t>(p) & (elem_bytes * 8 - 1)) return false;
  return true;
}
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
swiglu_bwd_kernel(const T* __restrict__ g, long long ldg, const T* __restrict__ u, long long ldu,
                  const T* __restrict__ dout, long long ldo, T* __restrict__ dg, long long lddg, T* __restrict__ du,
                  long long lddu, long long rows, int cols) {
  const long long n = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols;
    const int c = (int)(i % cols);
    const float gv = to_f32(g[r * ldg + c]), uv = to_f32(u[r * ldu + c]), d = to_f32(dout[r * ldo + c]);
    const float s = 1.0f / (1.0f + __expf(-gv));
    dg[r * lddg + c] = from_f32<T>(d * uv * s * (1.0f + gv * (1.0f - s)));
    du[r * lddu + c] = from_f32<T>(d * gv * s);
  }
}

// Row argmax over the first `cols` columns (first maximal index wins, like a left-to-right scan).
template <typename T>
__global__ void __launch_bounds__(256)
argmax_rows_kernel(const T* __restrict__ x, long long ld, long long* __restrict__ out, long long rows, int cols) {
  __shared__ float sv[256];
  __shared__ int si[256];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float v = to_f32(x[r * ld + c]);
      if (v > best || (v == best && c < bi)) { best = v; bi = c; }
    }
    sv[threadIdx.x] = best;
    si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
      if (threadIdx.x < s) {
        const float ov = sv[threadIdx.x + s];
        const int oi = si[threadIdx.x + s];
        if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) { sv[threadIdx.x] = ov; si[threadIdx.x] = oi; }
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) out[r] = si[0] == 0x7fffffff ? 0 : si[0];
    __syncthreads();
  }
}

// Temperature + top-k sampling, one CTA per row: k rounds of block argmax pick the k largest scaled logits (k <= 64),
// then thread 0 walks the CDF of their softmax with the uniform u[row]
// (reference sampler: lib/core/nn/gpt.dart:288-342).
template <typename T>
__global__ void __launch_bounds__(256)
topk_sample_kernel(const T* __restrict__ x, long long ld, const float* __restrict__ u, long long* __restrict__ out,
                   long long rows, int cols, int k, float temperature) {
  __shared__ float sv[256];
  __shared__ int si[256];
  __shared__ float top_v[64];
  __shared__ int top_i[64];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    for (int round = 0; round < k; ++round) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        bool taken = false;
        for (int j = 0; j < round; ++j) taken |= (top_i[j] == c);
        if (taken) continue;
        const float v = to_f32(x[r * ld + c]) / temperature;
        if (v > best || (v == best && c < bi)) { best = v; bi = c; }
      }
      sv[threadIdx.x] = best;
      si[threadIdx.x] = bi;
      __syncthreads();
      for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
          const float ov = sv[threadIdx.x + s];
          const int oi = si[threadIdx.x + s];
          if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) { sv[threadIdx.x] = ov; si[threadIdx.x] = oi; }
        }
        __syncthreads();
      }
      if (threadIdx.x == 0) { top_v[round] = sv[0]; top_i[round] = si[0]; }
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      const float m = top_v[0];
      float tot = 0.0f;
      for (int j = 0; j < k; ++j) tot += expf(top_v[j] - m);
      const float target = u[r] * tot;
      float acc = 0.0f;
      int pick = top_i[0];
      for (int j = 1; j < k; ++j) pick = top_i[j] > pick ? top_i[j] : pick;  // default: last kept index
      // Walk the kept entries in ascending index order, as the reference walks the vocabulary left to right.
      bool done = false;
      for (int rank = 0; rank < k && !done; ++rank) {
        for (int j = 0; j < k; ++j) {
          int smaller = 0;
          for (int q = 0; q < k; ++q) smaller += (top_i[q] < top_i[j]);
          if (smaller == rank) {
            acc += expf(top_v[j] - m);
            if (target <= acc) { pick = top_i[j]; done = true; }
            break;
          }
        }
      }
      out[r] = pick;
    }
    __syncthreads();
  }
}

// LC0 8x8 board unfold: in [B*64, C] (NHWC-flat) -> out [B*64, C*k*k], zero padding k/2, column = c*k*k + ky*k + kx
// (reference: lib/native/src/kernels/im2col.cuh:17-50).
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
im2col_nhwc_kernel(const T* __restrict__ in, T* __restrict__ out, int batch, int channels, int ksize, int board) {
  const int pad = ksize / 2;
  const long long kk = (long long)ksize * ksize;
  const long long row_len = channels * kk;
  const long long n = (long long)batch * board * board * row_len;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / row_len;
    const long long col = i % row_len;
    const int c = (int)(col / kk), kidx = (int)(col % kk);
    const int ky = kidx / ksize, kx = kidx % ksize;
    const int b = (int)(row / (board * board)), cell = (int)(row % (board * board));
    const int y = cell / board + ky - pad, x = cell % board + kx - pad;
    T v = from_f32<T>(0.0f);
    if (y >= 0 && y < board && x >= 0 && x < board) v = in[((long long)b * board * board + y * board + x) * channels + c];
    out[i] = v;
  }
}

// General convolution lowering.  x [B, C, H, W] -> cols [B*Ho*Wo, C*Kh*Kw] (column order (c, ky, kx), matching a
// [Cout, Cin, Kh, Kw] weight flattened to [Cout, Cin*Kh*Kw]); zero padding (reference: lib/core/nn/conv2d.dart:120-180).
struct ConvGeom {
  int B, C, H, W, Kh, Kw, stride, pad, Ho, Wo;
};
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
im2col_nchw_kernel(const T* __restrict__ x, T* __restrict__ cols, ConvGeom g) {
  const long long row_len = (long long)g.C * g.Kh * g.Kw;
  const long long n = (long long)g.B * g.Ho * g.Wo * row_len;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / row_len;
    const int col = (int)(i - row * row_len);
    const int kx = col % g.Kw, ky = (col / g.Kw) % g.Kh, c = col / (g.Kw * g.Kh);
    const int wo = (int)(row % g.Wo), ho = (int)((row / g.Wo) % g.Ho), b = (int)(row / ((long long)g.Wo * g.Ho));
    const int y = ho * g.stride - g.pad + ky, xx = wo * g.stride - g.pad + kx;
    T v = from_f32<T>(0.0f);
    if (y >= 0 && y < g.H && xx >= 0 && xx < g.W) v = x[(((long long)b * g.C + c) * g.H + y) * g.W + xx];
    cols[i] = v;
  }
}
// Adjoint of the lowering: dx[b, c, y, x] = sum over the (ky, kx, ho, wo) that read it.  Gather form, so no atomics and
// a fixed summation order.
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
col2im_nchw_kernel(const T* __restrict__ cols, T* __restrict__ dx, ConvGeom g) {
  const long long row_len = (long long)g.C * g.Kh * g.Kw;
  const long long n = (long long)g.B * g.C * g.H * g.W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int xx = (int)(i % g.W), y = (int)((i / g.W) % g.H);
    const int c = (int)((i / ((long long)g.W * g.H)) % g.C), b = (int)(i / ((long long)g.W * g.H * g.C));
    float acc = 0.0f;
    for (int ky = 0; ky < g.Kh; ++ky) {
      const int yy = y + g.pad - ky;
      if (yy < 0 || yy % g.stride) continue;
      const int ho = yy / g.stride;
      if (ho >= g.Ho) continue;
      for (int kx = 0; kx < g.Kw; ++kx) {
        const int xw = xx + g.pad - kx;
        if (xw < 0 || xw % g.stride) continue;
        const int wo = xw / g.stride;
        if (wo >= g.Wo) continue;
        const long long row = ((long long)b * g.Ho + ho) * g.Wo + wo;
        acc += to_f32(cols[row * row_len + ((long long)c * g.Kh + ky) * g.Kw + kx]);
      }
    }
    dx[i] = from_f32<T>(acc);
  }
}

// Image [B, C, H, W] -> patch rows [B * (H/P) * (W/P), P*P*C] with per-patch order (dy, dx, c): the input layout of the
// patch-projection GEMM (reference patch order: lib/core/data/image_folder_dataset.dart:180-205).
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(kEwThreads)
patchify_kernel(const TIn* __restrict__ img, TOut* __restrict__ out, int B, int C, int H, int W, int P) {
  const int gh = H / P, gw = W / P;
  const long long row_len = (long long)P * P * C;
  const long long n = (long long)B * gh * gw * row_len;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / row_len;
    const int col = (int)(i % row_len);
    const int c = col % C, dx = (col / C) % P, dy = col / (C * P);
    const int b = (int)(row / (gh * gw)), pr = (int)(row % (gh * gw));
    const int py = pr / gw, px = pr % gw;
    out[i] = from_f32<TOut>(to_f32(img[(((long long)b * C + c) * H + py * P + dy) * W + px * P + dx]));
  }
}

}  // namespace dptb

using namespace dptb;

#define DPTB_BY_DTYPE(dtype, CALL_BF16, CALL_F32) \
  do {                                            \
    if (dtype) { CALL_BF16; } else { CALL_F32; }  \
  } while (0)

extern "C" int dptb_binary(const void* a, const void* b, void* out, long long n, long long cols, int op, int bmode,
                           int dtype, void* stream) {
  if (n <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  DPTB_BY_DTYPE(dtype,
                (binary_kernel<__nv_bfloat16><<<ew_grid(n), kEwThreads, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, n, cols, op, bmode)),
                (binary_kernel<float><<<ew_grid(n), kEwThreads, 0, st>>>((const float*)a, (const float*)b, (float*)out, n, cols, op, bmode)));
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_unary(const void* x, void* out, long long n, int op, float param, int dtype, void* stream) {
  if (n <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  DPTB_BY_DTYPE(dtype,
                (unary_kernel<__nv_bfloat16><<<ew_grid(n), kEwThreads, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, op, param)),
                (unary_kernel<float><<<ew_grid(n), kEwThreads, 0, st>>>((const float*)x, (float*)out, n, op, param)));
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_unary_bwd(const void* x, const void* dy, void* dx, long long n, int op, float param, int dtype,
                              void* stream) {
  if (n <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  DPTB_BY_DTYPE(dtype,
                (unary_bwd_kernel<__nv_bfloat16><<<ew_grid(n), kEwThreads, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, n, op, param)),
                (unary_bwd_kernel<float><<<ew_grid(n), kEwThreads, 0, st>>>((const float*)x, (const float*)dy, (float*)dx, n, op, param)));
  return counted(1, (int)cudaGetLastError());
}
// partial: fp32 scratch of nparts * cols floats; out has `out_dtype` (0 fp32, 1 bf16).
extern "C" int dptb_colsum(const void* x, long long ld, void* out, float* partial, long long rows, int cols, int nparts,
                           int accumulate, int dtype, void* stream) {
  if (cols <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  if (nparts < 1) return kErrBadShape;
  if (dtype == 1 && (cols & 7) == 0 && (ld & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    dim3 vgrid((cols + 255) / 256, nparts);
    colsum_partial_vec8_kernel<<<vgrid, 256, 0, st>>>((const __nv_bfloat16*)x, ld, rows, cols, partial);
    DPTB_CUDA_OK(cudaGetLastError());
    colsum_final_wide_kernel<__nv_bfloat16><<<(cols + 31) / 32, 256, 0, st>>>(partial, nparts, cols, (__nv_bfloat16*)out, accumulate);
    return counted(2, (int)cudaGetLastError());
  }
  dim3 grid((cols + 63) / 64, nparts);
  DPTB_BY_DTYPE(dtype,
                (colsum_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ld, rows, cols, partial)),
                (colsum_partial_kernel<float><<<grid, 256, 0, st>>>((const float*)x, ld, rows, cols, partial)));
  DPTB_CUDA_OK(cudaGetLastError());
  DPTB_BY_DTYPE(dtype,
                (colsum_final_kernel<__nv_bfloat16><<<(cols + 255) / 256, 256, 0, st>>>(partial, nparts, cols, (__nv_bfloat16*)out, accumulate)),
                (colsum_final_kernel<float><<<(cols + 255) / 256, 256, 0, st>>>(partial, nparts, cols, (float*)out, accumulate)));
  return counted(2, (int)cudaGetLastError());
}
// partial: fp32 scratch of at least 148*16 floats.
extern "C" int dptb_sum_all(const void* x, long long n, float* out, float* partial, float scale, int dtype, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  const int parts = ew_grid(n);
  DPTB_BY_DTYPE(dtype,
                (sum_partial_kernel<__nv_bfloat16><<<parts, kEwThreads, 0, st>>>((const __nv_bfloat16*)x, n, partial)),
                (sum_partial_kernel<float><<<parts, kEwThreads, 0, st>>>((const float*)x, n, partial)));
  DPTB_CUDA_OK(cudaGetLastError());
  sum_final_kernel<<<1, 1024, 0, st>>>(partial, parts, out, scale);
  return counted(2, (int)cudaGetLastError());
}
extern "C" int dptb_transpose2d(const void* in, void* out, long long rows, long long cols, int dtype, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
  DPTB_BY_DTYPE(dtype,
                (transpose_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, rows, cols)),
                (transpose_kernel<float><<<grid, 256, 0, st>>>((const float*)in, (float*)out, rows, cols)));
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_copy2d(const void* src, long long lds, void* dst, long long ldd, long long rows, long long cols,
                           int dtype, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  DPTB_BY_DTYPE(dtype,
                (copy2d_kernel<__nv_bfloat16><<<ew_grid(rows * cols), kEwThreads, 0, st>>>((const __nv_bfloat16*)src, lds, (__nv_bfloat16*)dst, ldd, rows, cols)),
                (copy2d_kernel<float><<<ew_grid(rows * cols), kEwThreads, 0, st>>>((const float*)src, lds, (float*)dst, ldd, rows, cols)));
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_rope(const void* x, void* out, long long tokens, int heads, int head_dim, int rotary_dim,
                         int seq_len, int pos_start, float base, int inverse, int dtype, long long ld_in,
                         long long ld_out, const long long* positions, void* stream) {
  if (tokens <= 0) return 0;
  if (rotary_dim % 2 || rotary_dim > head_dim) return kErrBadShape;
  auto st = static_cast<cudaStream_t>(stream);
  const long long n = tokens * heads * (rotary_dim / 2);
  DPTB_BY_DTYPE(dtype,
                (rope_kernel<__nv_bfloat16><<<ew_grid(n), kEwThreads, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, tokens, heads, head_dim, rotary_dim, seq_len, pos_start, base, inverse, positions, ld_in, ld_out)),
                (rope_kernel<float><<<ew_grid(n), kEwThreads, 0, st>>>((const float*)x, (float*)out, tokens, heads, head_dim, rotary_dim, seq_len, pos_start, base, inverse, positions, ld_in, ld_out)));
  DPTB_CUDA_OK(cudaGetLastError());
  if (x != out && rotary_dim < head_dim) {
    const long long nt = tokens * heads * (head_dim - rotary_dim);
    DPTB_BY_DTYPE(dtype,
                  (rope_tail_kernel<__nv_bfloat16><<<ew_grid(nt), kEwThreads, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, tokens, heads, head_dim, rotary_dim, ld_in, ld_out)),
                  (rope_tail_kernel<float><<<ew_grid(nt), kEwThreads, 0, st>>>((const float*)x, (float*)out, tokens, heads, head_dim, rotary_dim, ld_in, ld_out)));
  }
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_dropout(const void* x, void* out, long long n, float p, unsigned long long seed,
                            unsigned long long offset, int dtype, void* stream) {
  if (n <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  DPTB_BY_DTYPE(dtype,
                (dropout_kernel<__nv_bfloat16><<<ew_grid(n), kEwThreads, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, p, seed, offset)),
                (dropout_kernel<float><<<ew_grid(n), kEwThreads, 0, st>>>((const float*)x, (float*)out, n, p, seed, offset)));
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_swiglu_fwd(const void* g, long long ldg, const void* u, long long ldu, void* out, long long ldo,
                               long long rows, int cols, int dtype, void* stream) {
  if (rows <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  if (vec8_ok(cols, {ldg, ldu, ldo}, {g, u, out}, dtype ? 2 : 4)) {
    const long long nv = rows * (cols >> 3);
    DPTB_BY_DTYPE(dtype,
                  (launch_k(swiglu_fwd_vec8_kernel<__nv_bfloat16>, dim3(ew_grid(nv)), dim3(kEwThreads), 0, st, (const __nv_bfloat16*)g, ldg, (const __nv_bfloat16*)u, ldu, (__nv_bfloat16*)out, ldo, rows, cols)),
                  (swiglu_fwd_vec8_kernel<float><<<ew_grid(nv), kEwThreads, 0, st>>>((const float*)g, ldg, (const float*)u, ldu, (float*)out, ldo, rows, cols)));
    return counted(1, (int)cudaGetLastError());
  }
  DPTB_BY_DTYPE(dtype,
                (swiglu_fwd_kernel<__nv_bfloat16><<<ew_grid(rows * cols), kEwThreads, 0, st>>>((const __nv_bfloat16*)g, ldg, (const __nv_bfloat16*)u, ldu, (__nv_bfloat16*)out, ldo, rows, cols)),
                (swiglu_fwd_kernel<float><<<ew_grid(rows * cols), kEwThreads, 0, st>>>((const float*)g, ldg, (const float*)u, ldu, (float*)out, ldo, rows, cols)));
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_swiglu_bwd(const void* g, long long ldg, const void* u, long long ldu, const void* dout,
                               long long ldo, void* dg, long long lddg, void* du, long long lddu, long long rows,
                               int cols, int dtype, void* stream) {
  if (rows <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  if (vec8_ok(cols, {ldg, ldu, ldo, lddg, lddu}, {g, u, dout, dg, du}, dtype ? 2 : 4)) {
    const long long nv = rows * (cols >> 3);
    DPTB_BY_DTYPE(dtype,
                  (swiglu_bwd_vec8_kernel<__nv_bfloat16><<<ew_grid(nv), kEwThreads, 0, st>>>((const __nv_bfloat16*)g, ldg, (const __nv_bfloat16*)u, ldu, (const __nv_bfloat16*)dout, ldo, (__nv_bfloat16*)dg, lddg, (__nv_bfloat16*)du, lddu, rows, cols)),
                  (swiglu_bwd_vec8_kernel<float><<<ew_grid(nv), kEwThreads, 0, st>>>((const float*)g, ldg, (const float*)u, ldu, (const float*)dout, ldo, (float*)dg, lddg, (float*)du, lddu, rows, cols)));
    return counted(1, (int)cudaGetLastError());
  }
  DPTB_BY_DTYPE(dtype,
                (swiglu_bwd_kernel<__nv_bfloat16><<<ew_grid(rows * cols), kEwThreads, 0, st>>>((const __nv_bfloat16*)g, ldg, (const __nv_bfloat16*)u, ldu, (const __nv_bfloat16*)dout, ldo, (__nv_bfloat16*)dg, lddg, (__nv_bfloat16*)du, lddu, rows, cols)),
                (swiglu_bwd_kernel<float><<<ew_grid(rows * cols), kEwThreads, 0, st>>>((const float*)g, ldg, (const float*)u, ldu, (const float*)dout, ldo, (float*)dg, lddg, (float*)du, lddu, rows, cols)));
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_argmax_rows(const void* x, long long ld, long long* out, long long rows, int cols, int dtype,
                                void* stream) {
  if (rows <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = (int)(rows < 4096 ? rows : 4096);
  DPTB_BY_DTYPE(dtype,
                (argmax_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ld, out, rows, cols)),
                (argmax_rows_kernel<float><<<grid, 256, 0, st>>>((const float*)x, ld, out, rows, cols)));
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_topk_sample(const void* x, long long ld, const float* u, long long* out, long long rows, int cols,
                                int k, float temperature, int dtype, int reserved, void* stream) {
  (void)reserved;
  if (rows <= 0) return 0;
  if (k < 1 || k > 64 || temperature <= 0.0f) return kErrBadShape;
  if (k > cols) k = cols;
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = (int)(rows < 4096 ? rows : 4096);
  DPTB_BY_DTYPE(dtype,
                (topk_sample_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ld, u, out, rows, cols, k, temperature)),
                (topk_sample_kernel<float><<<grid, 256, 0, st>>>((const float*)x, ld, u, out, rows, cols, k, temperature)));
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_im2col_nhwc(const void* in, void* out, int batch, int channels, int ksize, int board, int dtype,
                                void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  const long long n = (long long)batch * board * board * channels * ksize * ksize;
  if (n <= 0) return 0;
  DPTB_BY_DTYPE(dtype,
                (im2col_nhwc_kernel<__nv_bfloat16><<<ew_grid(n), kEwThreads, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, batch, channels, ksize, board)),
                (im2col_nhwc_kernel<float><<<ew_grid(n), kEwThreads, 0, st>>>((const float*)in, (float*)out, batch, channels, ksize, board)));
  return counted(1, (int)cudaGetLastError());
}
// direction 0: x -> cols (im2col); 1: cols -> dx (col2im, the adjoint).
extern "C" int dptb_conv_lower(const void* src, void* dst, int B, int C, int H, int W, int Kh, int Kw, int stride,
                               int pad, int direction, int dtype, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  if (B <= 0 || C <= 0 || Kh <= 0 || Kw <= 0 || stride <= 0 || pad < 0) return kErrBadShape;
  const int Ho = (H + 2 * pad - Kh) / stride + 1, Wo = (W + 2 * pad - Kw) / stride + 1;
  if (H + 2 * pad < Kh || W + 2 * pad < Kw || Ho <= 0 || Wo <= 0) return kErrBadShape;
  ConvGeom g{B, C, H, W, Kh, Kw, stride, pad, Ho, Wo};
  if (direction == 0) {
    const long long n = (long long)B * Ho * Wo * C * Kh * Kw;
    DPTB_BY_DTYPE(dtype,
                  (im2col_nchw_kernel<__nv_bfloat16><<<ew_grid(n), kEwThreads, 0, st>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, g)),
                  (im2col_nchw_kernel<float><<<ew_grid(n), kEwThreads, 0, st>>>((const float*)src, (float*)dst, g)));
  } else {
    const long long n = (long long)B * C * H * W;
    DPTB_BY_DTYPE(dtype,
                  (col2im_nchw_kernel<__nv_bfloat16><<<ew_grid(n), kEwThreads, 0, st>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, g)),
                  (col2im_nchw_kernel<float><<<ew_grid(n), kEwThreads, 0, st>>>((const float*)src, (float*)dst, g)));
  }
  return counted(1, (int)cudaGetLastError());
}
// in_dtype / out_dtype packed as dtype = in + 2*out.
extern "C" int dptb_patchify(const void* img, void* out, int B, int C, int H, int W, int P, int dtype, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  if (H % P || W % P) return kErrBadShape;
  const long long n = (long long)B * C * H * W;
  if (n <= 0) return 0;
  const int in_bf = dtype & 1, out_bf = (dtype >> 1) & 1;
  if (in_bf && out_bf) patchify_kernel<__nv_bfloat16, __nv_bfloat16><<<ew_grid(n), kEwThreads, 0, st>>>((const __nv_bfloat16*)img, (__nv_bfloat16*)out, B, C, H, W, P);
  else if (!in_bf && out_bf) patchify_kernel<float, __nv_bfloat16><<<ew_grid(n), kEwThreads, 0, st>>>((const float*)img, (__nv_bfloat16*)out, B, C, H, W, P);
  else if (!in_bf && !out_bf) patchify_kernel<float, float><<<ew_grid(n), kEwThreads, 0, st>>>((const float*)img, (float*)out, B, C, H, W, P);
  else patchify_kernel<__nv_bfloat16, float><<<ew_grid(n), kEwThreads, 0, st>>>((const __nv_bfloat16*)img, (float*)out, B, C, H, W, P);
  return counted(1, (int)cudaGetLastError());
}
