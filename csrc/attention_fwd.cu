// Flash-style attention forward on tcgen05 tensor cores with TMEM accumulators (bf16 in, fp32 softmax).
//
// Replaces the reference's per-head, per-batch-element chain  matmul -> scale -> +mask -> softmax -> matmul
// that materialises every [N, N] score matrix (reference: lib/core/tensor/attention.dart:39-53,
// lib/core/nn/attention/multi_head_attention.dart:181-235).  Nothing of size N x N touches HBM here.
//
// Operands are read in place from token-major projection outputs: element (b, s, head, d) of Q sits at
// q[(b*Sq + s) * ldq + head*hd + d] (same for K, V with their own leading dimensions), so a fused QKV GEMM
// output needs no split / permute, and O is written as [B*Sq, Hq*hd] ready for the output projection.
// Grouped-query attention: query head h reads KV head h / (Hq / Hkv).
//
// One CTA owns NQ query tiles of 128 rows of one (batch, head) and walks the KV sequence in tiles of 128 keys:
//   warps 0-3 / 4-7  softmax warpgroups, one per query tile, one thread per query row: pull the whole S row (128
//                    scores) from TMEM into registers in one go and hand the S columns straight back to the tensor
//                    core, so S_t(j+1) = Q_t K_{j+1}^T is computed while this tile's softmax runs; then max / exp2 /
//                    sum and P (bf16) into shared memory in the tensor core's K-major swizzled layout
//   warp 8           TMA producer (Q once, K / V through rings)
//   warp 9           MMA issuer: S_t = Q_t K_j^T, and O_t += P_t V_j accumulated in TMEM
// The output accumulator never leaves TMEM during the loop.  The running maximum is lazy: a row keeps exponentiating
// against an older maximum until the true one has grown by more than 8 (a factor 256 of headroom in fp32 / bf16);
// only then (decided per warp) O is pulled out, rescaled and stored back, which after the first tiles is rare.
#include <cuda_bf16.h>

#include "common/host.h"
#include "common/ptx.cuh"

namespace dptb {

struct AttnFwdParams {
  __nv_bfloat16* o;       // [B*Sq, ldo]
  float* lse;             // [B, Hq, Sq] natural-log log-sum-exp of the scaled scores (may be null)
  long long ldo;
  int B, Sq, Sk, Hq, Hkv;
  int causal;
  int q_offset;           // key j is visible to query i when j <= i + q_offset (causal)
  float scale_log2;       // softmax scale * log2(e)
  int num_q_blocks;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr int kAttnBM = 128;   // query rows per tile
constexpr int kAttnBN = 128;   // keys per tile
constexpr int kAttnThreads = 384;   // two softmax warpgroups + one warpgroup holding the TMA and MMA warps
// Registers per thread after the hand-over.  The CTA starts with 384 x 168 registers and the pool does not grow:
// 2 x 128 x 216 + 128 x 72 = 384 x 168, so the increase can always be satisfied once the producers have shrunk.
constexpr int kSoftmaxRegs = 216;
constexpr int kProducerRegs = 72;
static_assert(2 * 128 * kSoftmaxRegs + 128 * kProducerRegs <= kAttnThreads * 168, "register hand-over must balance");
constexpr float kLazyMaxSlack = 8.0f;   // log2 units a row's maximum may grow before O is rescaled

// Opt-in phase timers (compile with -DDPTB_ATTN_PROFILE): SM clock cycles that thread 0 of softmax warpgroup 0 spent,
// summed per CTA:  [0] waiting for S   [1] S: TMEM -> registers   [2] mask + maximum   [3] rescale of O
// [4] waiting for the previous P.V   [5] exp2 + pack + shared-memory stores   [6] whole loop   [7] KV tiles
#ifdef DPTB_ATTN_PROFILE
__device__ unsigned long long g_attn_prof[8];
#define ATTN_PROF_MARK(t) const long long t = clock64()
#define ATTN_PROF_ADD(slot, t0, t1) prof_acc[slot] += (t1) - (t0)
#else
#define ATTN_PROF_MARK(t)
#define ATTN_PROF_ADD(slot, t0, t1)
#endif

template <int HD, int NQ, int KST, int VST>
struct AttnFwdSmem {
  static constexpr int kQBytes = kAttnBM * HD * 2;
  static constexpr int kKVBytes = kAttnBN * HD * 2;
  static constexpr int kPBytes = kAttnBM * kAttnBN * 2;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + NQ * kQBytes;
  static constexpr int kVOff = kKOff + KST * kKVBytes;
  static constexpr int kPOff = kVOff + VST * kKVBytes;
  static constexpr int kBarOff = kPOff + NQ * kPBytes;
  static constexpr int kNumBars = NQ + 2 * KST + 2 * VST + 4 * NQ + 1;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16 + 1024;
  static_assert(kTotal <= 227 * 1024, "attention forward: shared memory budget");
};

template <int HD, int NQ, int KST, int VST>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using L = AttnFwdSmem<HD, NQ, KST, VST>;
  constexpr int kChunks = HD / 64;            // 64-column (128-byte) chunks per head row
  constexpr int TMEM_COLS = 512;
  constexpr int kSCol = 0;                    // S_t at columns [t*128, t*128+128)
  constexpr int kOCol = 256;                  // O_t at columns [256 + t*HD, ...)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;                          // [NQ]
  uint64_t* k_full = q_full + NQ;                   // [KST]
  uint64_t* k_empty = k_full + KST;
  uint64_t* v_full = k_empty + KST;                 // [VST]
  uint64_t* v_empty = v_full + VST;
  uint64_t* s_full = v_empty + VST;                 // [NQ] S_t(j) is in TMEM
  uint64_t* s_empty = s_full + NQ;                  // [NQ] S_t(j) has been copied to registers
  uint64_t* p_full = s_empty + NQ;                  // [NQ] P_t(j) is in shared memory (and O_t is rescaled)
  uint64_t* o_full = p_full + NQ;                   // [NQ] O_t += P_t(j) V_j has completed
  uint64_t* drain_bar = o_full + NQ;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Heavy (late) query blocks first when causal.
  const int qb = p.causal ? (p.num_q_blocks - 1 - (int)blockIdx.x) : (int)blockIdx.x;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q_row0 = qb * (NQ * kAttnBM);

  // Number of KV tiles each query tile needs.
  int n_tiles[NQ];
  int n_max = 0;
#pragma unroll
  for (int t = 0; t < NQ; ++t) {
    const int r0 = q_row0 + t * kAttnBM;
    int n = 0;
    if (r0 < p.Sq) {
      int last_key = p.Sk - 1;
      if (p.causal) {
        const int r_last = min(r0 + kAttnBM - 1, p.Sq - 1);
        last_key = min(last_key, r_last + p.q_offset);
      }
      n = last_key >= 0 ? last_key / kAttnBN + 1 : 0;
    }
    n_tiles[t] = n;
    n_max = max(n_max, n);
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 9) {
    if (lane == 0) {
      for (int t = 0; t < NQ; ++t) {
        mbar_init(&q_full[t], 1);
        mbar_init(&s_full[t], 1);
        mbar_init(&s_empty[t], kAttnBM);
        mbar_init(&p_full[t], kAttnBM);
        mbar_init(&o_full[t], 1);
      }
      for (int s = 0; s < KST; ++s) {
        mbar_init(&k_full[s], 1);
        mbar_init(&k_empty[s], 1);
      }
      for (int s = 0; s < VST; ++s) {
        mbar_init(&v_full[s], 1);
        mbar_init(&v_empty[s], 1);
      }
      mbar_init(drain_bar, 1);
      mbar_fence_init();
    }
    __syncwarp();
    tmem_alloc<TMEM_COLS>(tmem_slot);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  static_assert(NQ == 2, "warp roles assume two softmax warpgroups");
  if (warp >= 8) {
    warpgroup_reg_dec<kProducerRegs>();
  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int t = 0; t < NQ; ++t) {
        if (n_tiles[t] == 0) continue;
        mbar_arrive_expect_tx(&q_full[t], L::kQBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(smem + L::kQOff + t * L::kQBytes + c * (kAttnBM * 128), &tmQ, &q_full[t], head * HD + c * 64,
                      q_row0 + t * kAttnBM, batch);
      }
      int k_issued = 0, v_issued = 0;
      for (int j = 0; j < n_max; ++j) {
        const int ks = j % KST, vs = j % VST;
        if (!mbar_wait(&k_empty[ks], ((j / KST) & 1) ^ 1, abort_flag, kWaitEmptyTimeout)) break;
        mbar_arrive_expect_tx(&k_full[ks], L::kKVBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(smem + L::kKOff + ks * L::kKVBytes + c * (kAttnBN * 128), &tmK, &k_full[ks],
                      kv_head * HD + c * 64, j * kAttnBN, batch);
        k_issued = j + 1;
        if (!mbar_wait(&v_empty[vs], ((j / VST) & 1) ^ 1, abort_flag, kWaitEmptyTimeout)) break;
        mbar_arrive_expect_tx(&v_full[vs], L::kKVBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(smem + L::kVOff + vs * L::kKVBytes + c * (kAttnBN * 128), &tmV, &v_full[vs],
                      kv_head * HD + c * 64, j * kAttnBN, batch);
        v_issued = j + 1;
      }
      if (*abort_flag) {
        // Wait (bounded) for copies that may still be landing in this CTA's shared memory.
        const uint64_t t0 = global_timer_ns();
        for (int t = 0; t < NQ; ++t)
          while (n_tiles[t] && !mbar_try_wait(&q_full[t], 0) && global_timer_ns() - t0 < kWaitLimitNs / 4) {}
        for (int j = max(0, k_issued - KST); j < k_issued; ++j)
          while (!mbar_try_wait(&k_full[j % KST], (j / KST) & 1) && global_timer_ns() - t0 < kWaitLimitNs / 4) {}
        for (int j = max(0, v_issued - VST); j < v_issued; ++j)
          while (!mbar_try_wait(&v_full[j % VST], (j / VST) & 1) && global_timer_ns() - t0 < kWaitLimitNs / 4) {}
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kAttnBM, kAttnBN, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(kAttnBM, HD, false, true);
      bool issued_any = false;
      bool ok = true;
      auto issue_s = [&](int t, int j) {
        const uint32_t qa = smem_u32(smem + L::kQOff + t * L::kQBytes);
        const uint32_t kb = smem_u32(smem + L::kKOff + (j % KST) * L::kKVBytes);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * (kAttnBM * 128) + (kk % 4) * 32;
          umma_bf16(tmem_base + kSCol + t * kAttnBN, make_smem_desc(qa + off, 16, 1024),
                    make_smem_desc(kb + off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&s_full[t]);
        issued_any = true;
      };
      // Prologue: S_t(0) for every query tile.
      if (n_max > 0) {
        ok = mbar_wait(&k_full[0], 0, abort_flag, kWaitFullTimeout);
        for (int t = 0; t < NQ && ok; ++t) {
          if (n_tiles[t] == 0) continue;
          ok = mbar_wait(&q_full[t], 0, abort_flag, kWaitFullTimeout);
          if (!ok) break;
          tc_fence_after_sync();
          issue_s(t, 0);
        }
        if (ok) umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_max && ok; ++j) {
        // (a) S_t(j+1) as soon as the softmax warpgroup has copied S_t(j) out of TMEM.
        if (j + 1 < n_max) {
          const int ks1 = (j + 1) % KST;
          ok = mbar_wait(&k_full[ks1], ((j + 1) / KST) & 1, abort_flag, kWaitFullTimeout);
          for (int t = 0; t < NQ && ok; ++t) {
            if (j + 1 >= n_tiles[t]) continue;
            ok = mbar_wait(&s_empty[t], j & 1, abort_flag, kWaitTmemEmptyTimeout);
            if (!ok) break;
            tc_fence_after_sync();
            issue_s(t, j + 1);
          }
          if (!ok) break;
          umma_commit(&k_empty[ks1]);
        }
        // (b) O_t += P_t(j) V_j once P_t(j) is in shared memory.
        const int vs = j % VST;
        ok = mbar_wait(&v_full[vs], (j / VST) & 1, abort_flag, kWaitFullTimeout);
        for (int t = 0; t < NQ && ok; ++t) {
          if (j >= n_tiles[t]) continue;
          ok = mbar_wait(&p_full[t], j & 1, abort_flag, kWaitFlagTimeout);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t pa = smem_u32(smem + L::kPOff + t * L::kPBytes);
          const uint32_t vb = smem_u32(smem + L::kVOff + vs * L::kKVBytes);
#pragma unroll
          for (int kk = 0; kk < kAttnBN / 16; ++kk) {
            const uint32_t aoff = (kk / 4) * (kAttnBM * 128) + (kk % 4) * 32;
            umma_bf16(tmem_base + kOCol + t * HD, make_smem_desc(pa + aoff, 16, 1024),
                      make_smem_desc(vb + kk * 2048, kAttnBN * 128, 1024), idesc_o, (j != 0 || kk != 0) ? 1u : 0u);
          }
          umma_commit(&o_full[t]);
          issued_any = true;
        }
        if (!ok) break;
        umma_commit(&v_empty[vs]);
      }
      if (*abort_flag && issued_any) {
        umma_commit(drain_bar);
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < kWaitLimitNs / 4) {}
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    warpgroup_reg_inc<kSoftmaxRegs>();
    const int t = warp >> 2;
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const int q_row = q_row0 + t * kAttnBM + row_in_tile;         // row inside the sequence
    const int n = n_tiles[t];
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t s_addr = lane_addr + kSCol + t * kAttnBN;
    const uint32_t o_addr = lane_addr + kOCol + t * HD;
    uint8_t* p_tile = smem + L::kPOff + t * L::kPBytes;

    float m_use = -INFINITY;   // the maximum the stored exponentials are relative to (lags the true maximum)
    float l_run = 0.0f;
    const int key_limit = p.causal ? min(p.Sk - 1, q_row + p.q_offset) : p.Sk - 1;  // last visible key of this row
    bool ok = true;
#ifdef DPTB_ATTN_PROFILE
    long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const long long prof_begin = clock64();
#endif

    for (int j = 0; j < n && ok; ++j) {
      ATTN_PROF_MARK(pt0);
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[t], j & 1, abort_flag, kWaitTmemFullTimeout));
      if (!ok) break;
      ATTN_PROF_MARK(pt1);
      tc_fence_after_sync();
      uint32_t s[kAttnBN];
#pragma unroll
      for (int c = 0; c < kAttnBN / 32; ++c) tmem_ld_32x32(s_addr + c * 32, reinterpret_cast<uint32_t(&)[32]>(s[c * 32]));
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&s_empty[t]);   // the tensor core may overwrite S_t with the next tile's scores
      ATTN_PROF_MARK(pt2);

      const int key0 = j * kAttnBN;
      if (key0 + kAttnBN - 1 > key_limit) {   // per-thread; no warp-level operation inside
#pragma unroll
        for (int i = 0; i < kAttnBN; ++i)
          if (key0 + i > key_limit) s[i] = 0xff800000u;   // -inf
      }
      // three-input maxima: half the instructions of the two-input form
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < kAttnBN; i += 8) {
        mx0 = fmax3(mx0, __uint_as_float(s[i + 0]), __uint_as_float(s[i + 1]));
        mx1 = fmax3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
        mx2 = fmax3(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
        mx3 = fmax3(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
      }
      const float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      ATTN_PROF_MARK(pt3);
      // Lazy maximum: move it only when some row of this warp outgrew its old one by more than the slack (the first
      // finite tile always does: -inf + slack = -inf).  Rows that move rescale what they have accumulated so far.
      if (__any_sync(0xffffffffu, m_tile > m_use + kLazyMaxSlack)) {
        const float m_new = fmaxf(m_use, m_tile);
        const float alpha = (m_new == -INFINITY) ? 1.0f : fast_exp2(m_use - m_new);   // m_use = -inf -> 0
        if (j > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(&o_full[t], (j - 1) & 1, abort_flag, kWaitTmemFullTimeout));
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(o_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(o_addr + c * 32, r);
          }
          tmem_st_wait();
        }
        l_run *= alpha;
        m_use = m_new;
      }
      const float m_sub = (m_use == -INFINITY) ? 0.0f : m_use;
      ATTN_PROF_MARK(pt4);
      // The previous P_t must have been consumed before it is overwritten (it nearly always has been by now).
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&o_full[t], (j - 1) & 1, abort_flag, kWaitTmemFullTimeout));
        if (!ok) break;
      }
      ATTN_PROF_MARK(pt5);
      // Probabilities -> bf16 -> shared memory (K-major, 128-byte swizzle), row sum.
      float l0 = 0.0f, l1 = 0.0f, l2 = 0.0f, l3 = 0.0f;
#pragma unroll
      for (int c = 0; c < kAttnBN / 32; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          // (Computing half of the exponentials as cubic polynomials on the FMA pipe was measured slower here: 117 us
          // against 102 us at B16 H12 S1024 hd64; the softmax warps are bound by issue slots, not by the
          // special-function unit.  Taking the exponentials two at a time in bf16, ex2.approx.bf16x2, was slower as
          // well, 115 us, for the unpacking its row sum needs.)
          const float a = fast_exp2(fmaf(__uint_as_float(s[c * 32 + i + 0]), p.scale_log2, -m_sub));
          const float b = fast_exp2(fmaf(__uint_as_float(s[c * 32 + i + 1]), p.scale_log2, -m_sub));
          const float e = fast_exp2(fmaf(__uint_as_float(s[c * 32 + i + 2]), p.scale_log2, -m_sub));
          const float f = fast_exp2(fmaf(__uint_as_float(s[c * 32 + i + 3]), p.scale_log2, -m_sub));
          l0 += a; l1 += b; l2 += e; l3 += f;
          packed[(i >> 1) + 0] = pack_bf16x2(a, b);
          packed[(i >> 1) + 1] = pack_bf16x2(e, f);
        }
        // 32 keys = 64 bytes = four 16-byte chunks of this row, in 64-key block (c / 2), at chunk (c % 2) * 4 + i.
        uint8_t* blk = p_tile + (c >> 1) * (kAttnBM * 128);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t chunk = (uint32_t)((c & 1) * 4 + i) ^ (uint32_t)(row_in_tile & 7);
          *reinterpret_cast<uint4*>(blk + row_in_tile * 128 + chunk * 16) =
              make_uint4(packed[i * 4 + 0], packed[i * 4 + 1], packed[i * 4 + 2], packed[i * 4 + 3]);
        }
      }
      l_run += (l0 + l1) + (l2 + l3);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&p_full[t]);
      ATTN_PROF_MARK(pt6);
      ATTN_PROF_ADD(0, pt0, pt1);
      ATTN_PROF_ADD(1, pt1, pt2);
      ATTN_PROF_ADD(2, pt2, pt3);
      ATTN_PROF_ADD(3, pt3, pt4);
      ATTN_PROF_ADD(4, pt4, pt5);
      ATTN_PROF_ADD(5, pt5, pt6);
    }
#ifdef DPTB_ATTN_PROFILE
    if (threadIdx.x == 0) {
      prof_acc[6] = clock64() - prof_begin;
      prof_acc[7] = n;
      for (int i = 0; i < 8; ++i) atomicAdd(&g_attn_prof[i], (unsigned long long)prof_acc[i]);
    }
#endif
    if (ok && n > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(&o_full[t], (n - 1) & 1, abort_flag, kWaitTmemFullTimeout));
      if (ok) {
        tc_fence_after_sync();
        const bool live = q_row < p.Sq;
        // a row without any visible key keeps m_use = -inf (its polynomial exponentials are 2^-127, not 0)
        const bool any_key = l_run > 0.0f && m_use != -INFINITY;
        const float inv = any_key ? 1.0f / l_run : 0.0f;
        __nv_bfloat16* dst = p.o + ((long long)batch * p.Sq + (live ? q_row : 0)) * p.ldo + (long long)head * HD;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(o_addr + c * 32, r);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int d = 0; d < 32; d += 8) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(r[d + 0]) * inv, __uint_as_float(r[d + 1]) * inv);
              u.y = pack_bf16x2(__uint_as_float(r[d + 2]) * inv, __uint_as_float(r[d + 3]) * inv);
              u.z = pack_bf16x2(__uint_as_float(r[d + 4]) * inv, __uint_as_float(r[d + 5]) * inv);
              u.w = pack_bf16x2(__uint_as_float(r[d + 6]) * inv, __uint_as_float(r[d + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + d) = u;
            }
          }
        }
        tc_fence_before_sync();
        if (live && p.lse) {
          const float lse2 = any_key ? m_use + log2f(l_run) : -INFINITY;
          p.lse[((long long)batch * p.Hq + head) * p.Sq + q_row] = lse2 * 0.6931471805599453f;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

static int encode_tmap_seq(CUtensorMap* map, const void* base, int heads, int hd, int seq, int batch, long long ld,
                           int box_rows, long long batch_rows = 0) {
  if (batch_rows <= 0) batch_rows = seq;
  // dims: {heads*hd (contiguous), seq, batch}: rows past the end of a sequence read as zeros.
  const uint64_t dims[3] = {(uint64_t)heads * hd, (uint64_t)seq, (uint64_t)batch};
  const uint64_t strides[2] = {(uint64_t)ld * 2, (uint64_t)batch_rows * ld * 2};
  const uint32_t box[3] = {64, (uint32_t)box_rows, 1};
  return encode_tmap_nd_bf16(map, base, 3, dims, strides, box);
}

}  // namespace dptb

using namespace dptb;

struct DptbAttnFwdArgs {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;
  long long ldq, ldk, ldv, ldo;
  int B, Sq, Sk, Hq, Hkv, head_dim;
  int causal, q_offset;
  float scale;
  long long kv_batch_rows;  // rows between consecutive batches of K / V (a cache's capacity); 0 = Sk
};

template <int HD, int NQ, int KST, int VST>
static int attn_fwd_launch(const DptbAttnFwdArgs* a, cudaStream_t st) {
  using L = AttnFwdSmem<HD, NQ, KST, VST>;
  CUtensorMap tmQ, tmK, tmV;
  int rc = encode_tmap_seq(&tmQ, a->q, a->Hq, HD, a->Sq, a->B, a->ldq, kAttnBM);
  if (rc) return rc;
  rc = encode_tmap_seq(&tmK, a->k, a->Hkv, HD, a->Sk, a->B, a->ldk, kAttnBN, a->kv_batch_rows);
  if (rc) return rc;
  rc = encode_tmap_seq(&tmV, a->v, a->Hkv, HD, a->Sk, a->B, a->ldv, kAttnBN, a->kv_batch_rows);
  if (rc) return rc;
  AttnFwdParams p;
  p.o = static_cast<__nv_bfloat16*>(a->o);
  p.lse = a->lse;
  p.ldo = a->ldo;
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.causal = a->causal;
  p.q_offset = a->q_offset;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.num_q_blocks = (a->Sq + NQ * kAttnBM - 1) / (NQ * kAttnBM);
  auto kern = attn_fwd_kernel<HD, NQ, KST, VST>;
  DPTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
  dim3 grid(p.num_q_blocks, a->Hq, a->B);
  kern<<<grid, kAttnThreads, L::kTotal, st>>>(tmQ, tmK, tmV, p);
  return counted(1, (int)cudaGetLastError());
}

// Phase timers (see DPTB_ATTN_PROFILE): copies the 8 counters out and zeroes them; -5 when not compiled in.
extern "C" int dptb_attn_fwd_profile_read(unsigned long long* out) {
#ifdef DPTB_ATTN_PROFILE
  int rc = (int)cudaMemcpyFromSymbol(out, g_attn_prof, sizeof(unsigned long long) * 8);
  if (rc) return rc;
  static unsigned long long zeros[8];
  return (int)cudaMemcpyToSymbol(g_attn_prof, zeros, sizeof(zeros));
#else
  (void)out;
  return kErrUnsupported;
#endif
}

extern "C" int dptb_attn_fwd(const DptbAttnFwdArgs* a, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  if (a->B <= 0 || a->Sq <= 0 || a->Hq <= 0) return 0;
  if (a->Sk <= 0 || a->Hkv <= 0 || a->Hq % a->Hkv) return kErrBadShape;
  if ((a->ldq % 8) || (a->ldk % 8) || (a->ldv % 8) || (a->ldo % 8)) return kErrBadShape;
  if ((reinterpret_cast<uintptr_t>(a->o) & 15) != 0) return kErrBadShape;
  if (a->head_dim == 64) return attn_fwd_launch<64, 2, 2, 2>(a, st);
  if (a->head_dim == 128) return attn_fwd_launch<128, 2, 2, 1>(a, st);
  return kErrUnsupported;
}
