// Embedding gather (optionally fused with a learned position table) and its scatter-add backward.
//
// Out-of-range indices read as a zero row and are skipped in the backward, as in the reference
// (lib/native/src/kernels/embedding.cuh:19-48).  The backward comes in two forms: a sorted,
// segmented sum (one warp per distinct index, rows added in ascending order -> bit-reproducible) and an
// atomic form used when no sorted order is supplied.
#include "common/host.h"
#include "common/reduce.cuh"

namespace dptb {

// out[n, :] = table[idx[n], :] (+ pos_table[(pos_start + n % seq_len), :]).  One warp per row.
template <typename T>
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const T* __restrict__ table, long long vocab, const long long* __restrict__ idx,
                     const T* __restrict__ pos_table, long long pos_rows, int pos_start, int seq_len,
                     T* __restrict__ out, long long n, int D, int vec_ok) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r = warp0; r < n; r += nwarps) {
    const long long t = idx[r];
    const bool ok = t >= 0 && t < vocab;
    const long long ppos = pos_table ? (long long)pos_start + (seq_len > 0 ? r % seq_len : r) : 0;
    const bool pok = pos_table && ppos >= 0 && ppos < pos_rows;
    const T* src = table + (ok ? t : 0) * D;
    const T* psrc = pos_table ? pos_table + (pok ? ppos : 0) * D : nullptr;
    T* dst = out + r * D;
    if (vec_ok) {
      for (int c = lane * 8; c < D; c += 256) {
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (ok) Vec8<T>::load(src + c, v);
        if (pok) {
          float pv[8];
          Vec8<T>::load(psrc + c, pv);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += pv[j];
        }
        Vec8<T>::store(dst + c, v);
      }
    } else {
      for (int c = lane; c < D; c += 32) {
        float v = ok ? to_f32(src[c]) : 0.0f;
        if (pok) v += to_f32(psrc[c]);
        dst[c] = from_f32<T>(v);
      }
    }
  }
}

__device__ __forceinline__ void atomic_add_t(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add_t(__nv_bfloat16* p, float v) { atomicAdd(p, __float2bfloat16(v)); }

// dtable[idx[n], :] += dout[n, :] with atomics (order of equal indices not fixed).
template <typename T>
__global__ void __launch_bounds__(256)
embedding_bwd_atomic_kernel(T* __restrict__ dtable, long long vocab, const long long* __restrict__ idx,
                            const T* __restrict__ dout, long long n, int D) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r = warp0; r < n; r += nwarps) {
    const long long t = idx[r];
    if (t < 0 || t >= vocab) continue;
    for (int c = lane; c < D; c += 32) atomic_add_t(dtable + t * D + c, to_f32(dout[r * D + c]));
  }
}

// Sorted form: sorted_idx ascending, perm[i] = source row of sorted position i (stable order).  The warp that sits on
// the first position of a run of equal indices adds the whole run in order and does one read-modify-write.
template <typename T>
__global__ void __launch_bounds__(256)
embedding_bwd_sorted_kernel(T* __restrict__ dtable, long long vocab, const long long* __restrict__ sorted_idx,
                            const long long* __restrict__ perm, const T* __restrict__ dout, long long n, int D,
                            int vec_ok) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long i = warp0; i < n; i += nwarps) {
    const long long t = sorted_idx[i];
    if (t < 0 || t >= vocab) continue;
    if (i > 0 && sorted_idx[i - 1] == t) continue;  // not a run start
    long long end = i + 1;
    while (end < n && sorted_idx[end] == t) ++end;
    if (vec_ok) {
      // 16-byte accesses: a lane owns 8 consecutive features of the row, rows of the run are added in order
      for (int c = lane * 8; c < D; c += 256) {
        float acc[8];
        Vec8<T>::load(dtable + t * D + c, acc);
        for (long long k = i; k < end; ++k) {
          float v[8];
          Vec8<T>::load(dout + perm[k] * D + c, v);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += v[j];
        }
        Vec8<T>::store(dtable + t * D + c, acc);
      }
    } else {
      for (int c = lane; c < D; c += 32) {
        float acc = to_f32(dtable[t * D + c]);
        for (long long k = i; k < end; ++k) acc += to_f32(dout[perm[k] * D + c]);
        dtable[t * D + c] = from_f32<T>(acc);
      }
    }
  }
}

// Learned positions are an arange, so their gradient is a strided batch sum: dpos[p, :] += sum_b dout[b*S + (p - start), :].
template <typename T>
__global__ void __launch_bounds__(256)
pos_embedding_bwd_kernel(T* __restrict__ dpos, long long pos_rows, int pos_start, int seq_len, long long batch,
                         const T* __restrict__ dout, int D) {
  const long long total = (long long)seq_len * D;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long s = e / D;
    const int c = (int)(e % D);
    const long long p = s + pos_start;
    if (p < 0 || p >= pos_rows) continue;
    float acc = to_f32(dpos[p * D + c]);
    for (long long b = 0; b < batch; ++b) acc += to_f32(dout[(b * seq_len + s) * D + c]);
    dpos[p * D + c] = from_f32<T>(acc);
  }
}

static inline int warp_grid(long long n) {
  long long blocks = (n + 7) / 8;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace dptb

using namespace dptb;

extern "C" int dptb_embedding_fwd(const void* table, long long vocab, const long long* idx, const void* pos_table,
                                  long long pos_rows, int pos_start, int seq_len, void* out, long long n, int D,
                                  int dtype, void* stream) {
  if (n <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  const int vec_ok = (D % 8 == 0) && (((reinterpret_cast<uintptr_t>(table) | reinterpret_cast<uintptr_t>(pos_table) |
                                        reinterpret_cast<uintptr_t>(out)) & 15) == 0);
  if (dtype) embedding_fwd_kernel<__nv_bfloat16><<<warp_grid(n), 256, 0, st>>>((const __nv_bfloat16*)table, vocab, idx, (const __nv_bfloat16*)pos_table, pos_rows, pos_start, seq_len, (__nv_bfloat16*)out, n, D, vec_ok);
  else       embedding_fwd_kernel<float><<<warp_grid(n), 256, 0, st>>>((const float*)table, vocab, idx, (const float*)pos_table, pos_rows, pos_start, seq_len, (float*)out, n, D, vec_ok);
  return counted(1, (int)cudaGetLastError());
}
// sorted_idx / perm may be null: then the atomic form runs.
extern "C" int dptb_embedding_bwd(void* dtable, long long vocab, const long long* idx, const long long* sorted_idx,
                                  const long long* perm, const void* dout, long long n, int D, int dtype, void* stream) {
  if (n <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  if (sorted_idx && perm) {
    const int vec_ok = (D % 8 == 0) && (((reinterpret_cast<uintptr_t>(dtable) | reinterpret_cast<uintptr_t>(dout)) & 15) == 0);
    if (dtype) embedding_bwd_sorted_kernel<__nv_bfloat16><<<warp_grid(n), 256, 0, st>>>((__nv_bfloat16*)dtable, vocab, sorted_idx, perm, (const __nv_bfloat16*)dout, n, D, vec_ok);
    else       embedding_bwd_sorted_kernel<float><<<warp_grid(n), 256, 0, st>>>((float*)dtable, vocab, sorted_idx, perm, (const float*)dout, n, D, vec_ok);
  } else {
    if (dtype) embedding_bwd_atomic_kernel<__nv_bfloat16><<<warp_grid(n), 256, 0, st>>>((__nv_bfloat16*)dtable, vocab, idx, (const __nv_bfloat16*)dout, n, D);
    else       embedding_bwd_atomic_kernel<float><<<warp_grid(n), 256, 0, st>>>((float*)dtable, vocab, idx, (const float*)dout, n, D);
  }
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_pos_embedding_bwd(void* dpos, long long pos_rows, int pos_start, int seq_len, long long batch,
                                      const void* dout, int D, int dtype, void* stream) {
  if (seq_len <= 0 || batch <= 0) return 0;
  auto st = static_cast<cudaStream_t>(stream);
  const long long total = (long long)seq_len * D;
  int blocks = (int)((total + 255) / 256);
  if (blocks > sm_count() * 8) blocks = sm_count() * 8;
  if (dtype) pos_embedding_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((__nv_bfloat16*)dpos, pos_rows, pos_start, seq_len, batch, (const __nv_bfloat16*)dout, D);
  else       pos_embedding_bwd_kernel<float><<<blocks, 256, 0, st>>>((float*)dpos, pos_rows, pos_start, seq_len, batch, (const float*)dout, D);
  return counted(1, (int)cudaGetLastError());
}
