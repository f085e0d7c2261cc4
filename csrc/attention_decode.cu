// Decode-time attention over a KV cache (one or a few new query tokens per sequence) and the fused rotary + cache
// append that precedes it.
//
// The reference keeps per-head K / V tensors on the device, re-uploads the whole cache after appending one row on the
// host and materialises [1, T] score rows per head (reference: lib/core/nn/kv_cache.dart:22-84,
// lib/core/nn/attention/multi_head_attention.dart:160-235, lib/core/tensor/concat.dart:51-90).  Here the cache is one
// [B, capacity, Hkv * hd] buffer per layer, new rows are written in place by the kernel that also applies RoPE, and
// attention streams each KV row exactly once for all query heads that share it (grouped-query attention).
//
// attn_decode_kernel: grid (splits, Hkv, B * Sq).  A CTA owns one (sequence, query position, kv head) and a contiguous
// chunk of the keys; its 4 warps take 16-key rounds round-robin, each through a private two-stage cp.async ring in
// shared memory (the next round's K and V rows are in flight while this one is computed).  A key / value row is
// covered by hd/8 lanes with 16 bytes each, scores of the G = Hq / Hkv grouped heads are reduced with shuffles inside
// those lanes (packed fp32 multiply-adds), the softmax is computed per round and the round's probabilities are fetched
// back by shuffle for the P.V accumulation.  Partial (max, sum, acc) per warp are merged in shared memory and, when
// the keys are split across CTAs, through an fp32 workspace: the last CTA of a (query row, kv head) to finish merges
// the splits itself (arrival counter), so one kernel runs per call (attn_decode_merge_kernel remains for shapes beyond
// the counter table).
// The kernel is memory-bound by design: the roofline is the KV bytes over HBM bandwidth.
#include <cuda_bf16.h>

#include "common/host.h"
#include "common/ptx.cuh"
#include "common/reduce.cuh"

namespace dptb {

constexpr int kDecWarps = 4;
constexpr int kMaxGroup = 8;   // query heads per kv head

struct DecodeArgs {
  const __nv_bfloat16* q;    // [B * Sq, ldq], head h at columns [h * hd, (h + 1) * hd)
  const __nv_bfloat16* k;    // [B, cap, ldkv] rows; kv head g at columns [g * hd, ...)
  const __nv_bfloat16* v;
  __nv_bfloat16* o;          // [B * Sq, ldo]
  float* ws;                 // [B * Sq, Hkv, splits, G, hd + 2] when splits > 1
  long long ldq, ldkv, ldo;
  long long kv_batch_stride; // elements between consecutive sequences of the cache (cap * ldkv)
  int B, Sq, Sk, Hq, Hkv, splits;
  int q_offset;              // absolute position of query row 0 (causal: query i sees keys <= q_offset + i)
  float scale;
  const int* pos_ptr;        // when set: q_offset = *pos_ptr and Sk = q_offset + Sq (device-resident position, so a
                             // captured CUDA graph can be replayed as the sequence grows)
  int cap;                   // cache rows per sequence: no key at or beyond it is ever read
  int fused_merge;           // the last split CTA of a (query row, kv head) merges the partials itself
};

__device__ __forceinline__ void unpack_bf16x8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// Eight bf16 -> four packed fp32 pairs (operands of fma.rn.f32x2: half the multiply-add instructions of scalar code).
__device__ __forceinline__ void unpack_bf16x8_f2(const uint4& u, f32x2 (&f)[4]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) f[i] = f2_pack(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
}

// GP = grouped query heads padded to a power of two (heads >= G carry zero queries).  A key row is covered by
// LPK = HD / 8 lanes with 16 bytes each.  Every warp streams its keys in rounds of 16 through a private two-stage ring in
// shared memory filled by cp.async (16 bytes per lane and instruction): the K and V rows of the next round are in
// flight while this round is computed, so the loads of the resident warps overlap their arithmetic instead of
// alternating with it, and no register holds data in flight.  Within a round sub-group sg (LPK lanes) owns keys
// sg * KS + u, u < KS = LPK / 2; lane u of the sub-group ends up holding that key's scores, the round's softmax is two
// warp reductions per head and the probabilities are fetched back by shuffle for P.V.
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
constexpr int kDecRound = 16;    // keys per round of a warp

// Arrival counters of the split CTAs of one (query row, kv head): the last CTA to arrive merges the partials, so no
// second kernel runs.  Zero at load, reset by the merging CTA; launches that use them must not overlap on two streams.
constexpr int kDecCounters = 1 << 16;
__device__ unsigned int g_dec_counters[kDecCounters];
constexpr int kDecMaxFusedSplits = 64;

template <int HD, int GP>
__global__ void __launch_bounds__(kDecWarps * 32, GP <= 4 ? 3 : 2)
attn_decode_kernel(const DecodeArgs a) {
  constexpr int LPK = HD / 8;                // lanes per key
  constexpr int NSG = 32 / LPK;              // sub-groups per warp
  constexpr int KS = kDecRound / NSG;        // keys per sub-group and round
  constexpr int kStageChunks = kDecRound * LPK;            // 16-byte chunks of one K (or V) stage
  constexpr int kWarpChunks = 4 * kStageChunks;            // two stages of K and V
  extern __shared__ uint4 dec_ring[];
  pdl_wait();                // (programmatic dependent launch: no-ops in an ordinary launch)
  pdl_launch_dependents();
  const int split = blockIdx.x, g = blockIdx.y, bs = blockIdx.z;
  const int b = bs / a.Sq, sq = bs % a.Sq;
  const int G = a.Hq / a.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sl = lane & (LPK - 1), sg0 = lane & ~(LPK - 1);   // lane within the sub-group, first lane of the sub-group
  const int q_off = a.pos_ptr ? *a.pos_ptr : a.q_offset;
  const int sk = a.pos_ptr ? q_off + a.Sq : a.Sk;
  const int visible = min(min(sk, a.cap), q_off + sq + 1);     // causal limit for this query row
  const int per = (visible + a.splits - 1) / a.splits;
  const int j0 = split * per, j1 = min(visible, j0 + per);

  __shared__ float s_m[kDecWarps][GP], s_l[kDecWarps][GP];
  __shared__ float s_acc[kDecWarps][GP][HD];

  f32x2 qv[GP][4];
  const __nv_bfloat16* qrow = a.q + (long long)bs * a.ldq + (long long)g * G * HD + sl * 8;
  const f32x2 scale2 = f2_splat(a.scale);
#pragma unroll
  for (int h = 0; h < GP; ++h) {
    if (h < G) {
      unpack_bf16x8_f2(*reinterpret_cast<const uint4*>(qrow + h * HD), qv[h]);
#pragma unroll
      for (int e = 0; e < 4; ++e) qv[h][e] = f2_mul(qv[h][e], scale2);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) qv[h][e] = f2_splat(0.0f);
    }
  }
  float m[GP], l[GP];
  f32x2 acc[GP][4];
#pragma unroll
  for (int h = 0; h < GP; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[h][e] = f2_splat(0.0f);
  }
  const __nv_bfloat16* kb = a.k + (long long)b * a.kv_batch_stride + (long long)g * HD;
  const __nv_bfloat16* vb = a.v + (long long)b * a.kv_batch_stride + (long long)g * HD;
  uint4* ring = dec_ring + warp * kWarpChunks;   // [stage][K | V][16 rows][LPK chunks]
  const int sg = lane / LPK;
  const int rounds = (j1 - j0 + kDecRound - 1) / kDecRound;   // of this CTA; warp w takes rounds w, w + 4, ...
  // Rows past the end of the range are fetched from the last valid row (finite data) and masked in the softmax.
  auto issue = [&](int t, int stage) {
    const int key0 = j0 + t * kDecRound;
    uint4* dst = ring + stage * 2 * kStageChunks;
#pragma unroll
    for (int it = 0; it < kStageChunks / 32; ++it) {
      const int c = it * 32 + lane;
      const int key = min(key0 + c / LPK, j1 - 1);
      const long long off = (long long)key * a.ldkv + (c % LPK) * 8;
      cp_async_16(dst + c, kb + off);
      cp_async_16(dst + kStageChunks + c, vb + off);
    }
    cp_async_commit();
  };
  if (warp < rounds) issue(warp, 0);
  int it_local = 0;
  for (int t = warp; t < rounds; t += kDecWarps, ++it_local) {
    const int stage = it_local & 1;
    if (t + kDecWarps < rounds) {
      issue(t + kDecWarps, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncwarp();
    const uint4* ks = ring + stage * 2 * kStageChunks;
    const uint4* vs = ks + kStageChunks;
    // ---- scores: lane u of a sub-group keeps the scores of key sg * KS + u of this round
    float sc[GP];
#pragma unroll
    for (int h = 0; h < GP; ++h) sc[h] = -INFINITY;
#pragma unroll
    for (int u = 0; u < KS; ++u) {
      f32x2 kf[4];
      unpack_bf16x8_f2(ks[(sg * KS + u) * LPK + sl], kf);
#pragma unroll
      for (int h = 0; h < GP; ++h) {
        f32x2 d2 = f2_mul(qv[h][0], kf[0]);
#pragma unroll
        for (int e = 1; e < 4; ++e) d2 = f2_fma(qv[h][e], kf[e], d2);
        float dlo, dhi;
        f2_unpack(d2, dlo, dhi);
        float d = dlo + dhi;
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (sl == u) sc[h] = d;
      }
    }
    const bool live = sl < KS && j0 + t * kDecRound + sg * KS + sl < j1;
    // ---- round softmax statistics and rescale
    float p[GP];
#pragma unroll
    for (int h = 0; h < GP; ++h) {
      const float s = live ? sc[h] : -INFINITY;
      const float nm = fmaxf(m[h], warp_max(s));
      const float corr = __expf(m[h] - nm);             // 0 on the first round (m = -inf)
      p[h] = live ? __expf(s - nm) : 0.0f;
      l[h] = l[h] * corr + warp_sum(p[h]);
      m[h] = nm;
      const f32x2 corr2 = f2_splat(corr);
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[h][e] = f2_mul(acc[h][e], corr2);
    }
    // ---- P.V: every sub-group accumulates its own keys; the sub-groups are folded once at the end
#pragma unroll
    for (int u = 0; u < KS; ++u) {
      f32x2 vf[4];
      unpack_bf16x8_f2(vs[(sg * KS + u) * LPK + sl], vf);
#pragma unroll
      for (int h = 0; h < GP; ++h) {
        const f32x2 pj = f2_splat(__shfl_sync(0xffffffffu, p[h], sg0 + u));
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[h][e] = f2_fma(pj, vf[e], acc[h][e]);
      }
    }
    __syncwarp();   // every lane has read this stage before the load two rounds ahead overwrites it
  }
  // ---- fold the sub-groups of the warp, then the warps of the CTA (fixed order)
#pragma unroll
  for (int h = 0; h < GP; ++h) {
    float af[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) f2_unpack(acc[h][e], af[2 * e], af[2 * e + 1]);
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
      for (int o = 16; o >= LPK; o >>= 1) af[e] += __shfl_xor_sync(0xffffffffu, af[e], o);
    if (lane == 0) {
      s_m[warp][h] = m[h];
      s_l[warp][h] = l[h];
    }
    if (lane < LPK) {
#pragma unroll
      for (int e = 0; e < 8; ++e) s_acc[warp][h][lane * 8 + e] = af[e];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    const int h = idx / HD, d = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, s_m[w][h]);
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float c = s_m[w][h] == -INFINITY ? 0.0f : __expf(s_m[w][h] - mm);
      ll += s_l[w][h] * c;
      oo += s_acc[w][h][d] * c;
    }
    if (a.splits == 1) {
      a.o[(long long)bs * a.ldo + (long long)(g * G + h) * HD + d] = __float2bfloat16(ll > 0.0f ? oo / ll : 0.0f);
    } else {
      float* w = a.ws + ((((long long)bs * a.Hkv + g) * a.splits + split) * G + h) * (HD + 2);
      w[d] = oo;
      if (d == 0) {
        w[HD] = mm;
        w[HD + 1] = ll;
      }
    }
  }
  if (a.splits == 1 || !a.fused_merge) return;
  // ---- the last CTA of this (query row, kv head) to get here merges the splits (fixed order: deterministic)
  __shared__ unsigned int s_last;
  __shared__ float s_sm[kDecMaxFusedSplits][GP], s_sl[kDecMaxFusedSplits][GP];
  __threadfence();   // this thread's partials are visible device-wide before the CTA is counted
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int* ctr = &g_dec_counters[bs * a.Hkv + g];
    const unsigned int prev = atomicAdd(ctr, 1u);
    s_last = prev == (unsigned int)a.splits - 1u ? 1u : 0u;
    if (s_last) *ctr = 0u;   // everyone has arrived: ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* base = a.ws + (((long long)bs * a.Hkv + g) * a.splits) * G * (HD + 2);
  const long long sstride = (long long)G * (HD + 2);
  for (int i = threadIdx.x; i < a.splits * G; i += blockDim.x) {
    const int sp = i / G, h = i % G;
    const float* w = base + sp * sstride + (long long)h * (HD + 2);
    s_sm[sp][h] = __ldcg(w + HD);
    s_sl[sp][h] = __ldcg(w + HD + 1);
  }
  __syncthreads();
  // Every thread owns up to NO outputs (idx = thread + k * 128); the loads of all of them for two splits are issued
  // together, so the merge is a few round trips to L2 instead of one per (output, split).
  constexpr int NO = (GP * HD + kDecWarps * 32 - 1) / (kDecWarps * 32);
  float mm[NO], ll[NO], oo[NO];
  int hh[NO];
  const float* wp[NO];
#pragma unroll
  for (int k = 0; k < NO; ++k) {
    const int idx = threadIdx.x + k * (kDecWarps * 32);
    const int h = idx / HD < G ? idx / HD : 0;       // padded heads repeat head 0 and are not stored
    hh[k] = h;
    wp[k] = base + (long long)h * (HD + 2) + idx % HD;
    float m = -INFINITY;
    for (int sp = 0; sp < a.splits; ++sp) m = fmaxf(m, s_sm[sp][h]);
    mm[k] = m;
    ll[k] = 0.0f;
    oo[k] = 0.0f;
  }
  int sp = 0;
  for (; sp + 2 <= a.splits; sp += 2) {
    float v0[NO], v1[NO];
#pragma unroll
    for (int k = 0; k < NO; ++k) {
      v0[k] = __ldcg(wp[k] + sp * sstride);
      v1[k] = __ldcg(wp[k] + (sp + 1) * sstride);
    }
#pragma unroll
    for (int k = 0; k < NO; ++k) {
      const float m0 = s_sm[sp][hh[k]], m1 = s_sm[sp + 1][hh[k]];
      const float c0 = m0 == -INFINITY ? 0.0f : __expf(m0 - mm[k]);
      const float c1 = m1 == -INFINITY ? 0.0f : __expf(m1 - mm[k]);
      ll[k] += s_sl[sp][hh[k]] * c0 + s_sl[sp + 1][hh[k]] * c1;
      oo[k] += v0[k] * c0 + v1[k] * c1;
    }
  }
  if (sp < a.splits) {
#pragma unroll
    for (int k = 0; k < NO; ++k) {
      const float m0 = s_sm[sp][hh[k]];
      const float c0 = m0 == -INFINITY ? 0.0f : __expf(m0 - mm[k]);
      ll[k] += s_sl[sp][hh[k]] * c0;
      oo[k] += __ldcg(wp[k] + sp * sstride) * c0;
    }
  }
#pragma unroll
  for (int k = 0; k < NO; ++k) {
    const int idx = threadIdx.x + k * (kDecWarps * 32);
    if (idx / HD < G)
      a.o[(long long)bs * a.ldo + (long long)(g * G + idx / HD) * HD + idx % HD] =
          __float2bfloat16(ll[k] > 0.0f ? oo[k] / ll[k] : 0.0f);
  }
}

template <int HD>
__global__ void __launch_bounds__(128)
attn_decode_merge_kernel(const DecodeArgs a) {
  const int G = a.Hq / a.Hkv;
  const int hq = blockIdx.x, bs = blockIdx.y;
  const int g = hq / G, h = hq % G;
  const float* base = a.ws + (((long long)bs * a.Hkv + g) * a.splits * G + h) * (HD + 2);
  const long long stride = (long long)G * (HD + 2);
  float mm = -INFINITY;
  for (int s = 0; s < a.splits; ++s) mm = fmaxf(mm, base[s * stride + HD]);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float ll = 0.0f, oo = 0.0f;
    for (int s = 0; s < a.splits; ++s) {
      const float ms = base[s * stride + HD];
      const float c = ms == -INFINITY ? 0.0f : __expf(ms - mm);
      ll += base[s * stride + HD + 1] * c;
      oo += base[s * stride + d] * c;
    }
    a.o[(long long)bs * a.ldo + (long long)hq * HD + d] = __float2bfloat16(ll > 0.0f ? oo / ll : 0.0f);
  }
}

// Rotary embedding (half-split form) on the Q and K column blocks of a fused projection row, K / V written straight
// into the cache at their absolute positions.  Grid: one CTA per (row, head) group; threads over the head dimension.
//   qkv row layout: [Hq * hd | Hkv * hd | Hkv * hd];  q is rotated in place (the attention kernel reads it there).
template <int HD>
__global__ void __launch_bounds__(128)
rope_kv_append_kernel(__nv_bfloat16* __restrict__ qkv, long long ld, __nv_bfloat16* __restrict__ kc,
                      __nv_bfloat16* __restrict__ vc, long long ldkv, long long kv_batch_stride, int B, int S, int Hq,
                      int Hkv, int pos0, int rotary_dim, float base, int cap, const int* __restrict__ pos_ptr) {
  pdl_wait();                // (programmatic dependent launch: no-ops in an ordinary launch)
  pdl_launch_dependents();
  const int row = blockIdx.x;                // b * S + s
  const int b = row / S, s = row % S;
  const int pos = (pos_ptr ? *pos_ptr : pos0) + s;
  if (pos >= cap) return;
  __nv_bfloat16* r = qkv + (long long)row * ld;
  const int half = rotary_dim / 2;
  const int heads = Hq + 2 * Hkv;
  // Thread -> one pair index i (angle computed once) and a strided subset of the heads.
  constexpr int PAIRS = HD / 2;
  const int i = threadIdx.x % PAIRS, hg = threadIdx.x / PAIRS, hstep = blockDim.x / PAIRS;
  // pair (i, i + half) inside the rotary part; dims >= rotary_dim pass through as the pair
  // (rotary_dim + 2 (i - half), + 1), so that every element is visited exactly once
  int d0, d1;
  float cs = 1.0f, sn = 0.0f;
  if (i < half) {
    d0 = i;
    d1 = i + half;
    const float inv = powf(base, -2.0f * (float)i / (float)rotary_dim);
    sincosf((float)pos * inv, &sn, &cs);
  } else {
    d0 = rotary_dim + 2 * (i - half);
    d1 = d0 + 1;
  }
  for (int h = hg; h < heads; h += hstep) {
    __nv_bfloat16* src = r + (long long)h * HD;
    const float x0 = __bfloat162float(src[d0]), x1 = __bfloat162float(src[d1]);
    const bool is_v = h >= Hq + Hkv;
    const float y0 = is_v ? x0 : x0 * cs - x1 * sn;
    const float y1 = is_v ? x1 : x1 * cs + x0 * sn;
    if (h < Hq) {
      src[d0] = __float2bfloat16(y0);
      src[d1] = __float2bfloat16(y1);
    } else {
      const int g = is_v ? h - Hq - Hkv : h - Hq;
      __nv_bfloat16* dst = (is_v ? vc : kc) + (long long)b * kv_batch_stride + (long long)pos * ldkv + (long long)g * HD;
      dst[d0] = __float2bfloat16(y0);
      dst[d1] = __float2bfloat16(y1);
    }
  }
}

}  // namespace dptb

using namespace dptb;

struct DptbDecodeArgs {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* ws;
  long long ws_floats;
  long long ldq, ldkv, ldo, kv_batch_stride;
  int B, Sq, Sk, Hq, Hkv, head_dim, splits, q_offset;
  float scale;
  const int* pos_ptr;
  int cap;
};

// Floats of workspace needed for a given split count.
extern "C" long long dptb_attn_decode_ws_floats(int B, int Sq, int Hq, int head_dim, int splits) {
  return splits <= 1 ? 0 : (long long)B * Sq * Hq * splits * (head_dim + 2);
}
// Split count that fills the GPU once: three CTAs fit an SM (registers), and a grid beyond that runs a second, mostly
// empty wave, so the count is rounded DOWN to what is resident at once; at least 128 keys (one 32-key block per warp)
// per CTA.
static int decode_splits(int B, int Sq, int Hkv, int Sk, int head_dim) {
  const int base = B * Sq * Hkv;
  (void)head_dim;
  const int per_sm = 3;   // CTAs resident per SM (registers): see the kernel's launch bounds
  int s = (per_sm * sm_count()) / base;
  const int cap = (Sk + 127) / 128;
  if (s > cap) s = cap;
  if (s > 64) s = 64;
  return s < 1 ? 1 : s;
}
extern "C" int dptb_attn_decode_splits(int B, int Sq, int Hkv, int Sk) { return decode_splits(B, Sq, Hkv, Sk, 64); }
extern "C" int dptb_attn_decode_splits_hd(int B, int Sq, int Hkv, int Sk, int head_dim) {
  return decode_splits(B, Sq, Hkv, Sk, head_dim);
}

extern "C" int dptb_attn_decode(const DptbDecodeArgs* h, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  if (h->B <= 0 || h->Sq <= 0 || h->Sk <= 0) return 0;
  if (h->Hkv <= 0 || h->Hq % h->Hkv || h->Hq / h->Hkv > kMaxGroup) return kErrUnsupported;
  if (h->head_dim != 64 && h->head_dim != 128) return kErrUnsupported;
  // rows are read in 16-byte pieces
  if ((h->ldkv % 8) || (h->kv_batch_stride % 8) || (h->ldq % 8) || (reinterpret_cast<uintptr_t>(h->k) & 15) ||
      (reinterpret_cast<uintptr_t>(h->v) & 15) || (reinterpret_cast<uintptr_t>(h->q) & 15))
    return kErrBadShape;
  DecodeArgs a;
  a.q = static_cast<const __nv_bfloat16*>(h->q);
  a.k = static_cast<const __nv_bfloat16*>(h->k);
  a.v = static_cast<const __nv_bfloat16*>(h->v);
  a.o = static_cast<__nv_bfloat16*>(h->o);
  a.ws = h->ws;
  a.ldq = h->ldq; a.ldkv = h->ldkv; a.ldo = h->ldo; a.kv_batch_stride = h->kv_batch_stride;
  a.B = h->B; a.Sq = h->Sq; a.Sk = h->Sk; a.Hq = h->Hq; a.Hkv = h->Hkv;
  a.splits = h->splits < 1 ? 1 : h->splits;
  a.q_offset = h->q_offset; a.scale = h->scale;
  a.pos_ptr = h->pos_ptr; a.cap = h->cap > 0 ? h->cap : h->Sk;
  if (a.splits > 1 && (!a.ws || h->ws_floats < dptb_attn_decode_ws_floats(a.B, a.Sq, a.Hq, h->head_dim, a.splits)))
    return kErrTooLarge;
  dim3 grid(a.splits, a.Hkv, a.B * a.Sq);
  const int G = a.Hq / a.Hkv;
  a.fused_merge = (a.splits > 1 && a.splits <= kDecMaxFusedSplits && (long long)a.B * a.Sq * a.Hkv <= kDecCounters) ? 1 : 0;
  const int gp = G <= 1 ? 1 : G <= 2 ? 2 : G <= 4 ? 4 : 8;
  // ring: two stages of 16 K rows and 16 V rows per warp
#define DPTB_DEC(HDV, GPV)                                                                                            \
  do {                                                                                                                \
    constexpr int kRing = kDecWarps * 4 * kDecRound * HDV * 2;                                                        \
    static bool attr_set = false;                                                                                     \
    if (!attr_set) {                                                                                                  \
      DPTB_CUDA_OK(cudaFuncSetAttribute(attn_decode_kernel<HDV, GPV>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                        kRing));                                                                      \
      attr_set = true;                                                                                                \
    }                                                                                                                 \
    DPTB_CUDA_OK(launch_k(attn_decode_kernel<HDV, GPV>, grid, dim3(kDecWarps * 32), kRing, st, a));                   \
  } while (0)
  if (h->head_dim == 128) {
    if (gp == 1) DPTB_DEC(128, 1); else if (gp == 2) DPTB_DEC(128, 2); else if (gp == 4) DPTB_DEC(128, 4); else DPTB_DEC(128, 8);
  } else {
    if (gp == 1) DPTB_DEC(64, 1); else if (gp == 2) DPTB_DEC(64, 2); else if (gp == 4) DPTB_DEC(64, 4); else DPTB_DEC(64, 8);
  }
#undef DPTB_DEC
  DPTB_CUDA_OK(cudaGetLastError());
  if (a.splits > 1 && !a.fused_merge) {
    dim3 mg(a.Hq, a.B * a.Sq);
    if (h->head_dim == 128) attn_decode_merge_kernel<128><<<mg, 128, 0, st>>>(a);
    else                    attn_decode_merge_kernel<64><<<mg, 128, 0, st>>>(a);
    return counted(2, (int)cudaGetLastError());
  }
  return counted(1, (int)cudaGetLastError());
}

extern "C" int dptb_rope_kv_append(void* qkv, long long ld, void* kc, void* vc, long long ldkv,
                                   long long kv_batch_stride, int B, int S, int Hq, int Hkv, int head_dim, int pos0,
                                   int rotary_dim, float base, int cap, const int* pos_ptr, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  if (B <= 0 || S <= 0) return 0;
  if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1) || pos0 < 0 || (!pos_ptr && pos0 + S > cap))
    return kErrBadShape;
  auto* q = static_cast<__nv_bfloat16*>(qkv);
  auto* k = static_cast<__nv_bfloat16*>(kc);
  auto* v = static_cast<__nv_bfloat16*>(vc);
  if (head_dim == 128)
    DPTB_CUDA_OK(launch_k(rope_kv_append_kernel<128>, dim3(B * S), dim3(128), 0, st, q, ld, k, v, ldkv, kv_batch_stride, B, S, Hq, Hkv, pos0, rotary_dim, base, cap, pos_ptr));
  else if (head_dim == 64)
    DPTB_CUDA_OK(launch_k(rope_kv_append_kernel<64>, dim3(B * S), dim3(128), 0, st, q, ld, k, v, ldkv, kv_batch_stride, B, S, Hq, Hkv, pos0, rotary_dim, base, cap, pos_ptr));
  else
    return kErrUnsupported;
  return counted(1, (int)cudaGetLastError());
}
