// Flash-style attention backward on tcgen05 tensor cores (head_dim 64, bf16 in, fp32 accumulate).
//
// The reference obtains attention gradients by replaying its forward op chain through the autograd tape
// (matmul / transpose / softmax backward per head, reference: lib/core/tensor/attention.dart:39-53,
// lib/core/tensor/mat_mul.dart:56-74).  Here one kernel recomputes the probabilities tile by tile and produces
// dQ, dK and dV without any [N, N] tensor in HBM.
//
// One CTA owns one tile of 128 keys of one (batch, KV head) and loops over the query heads of its group and over the
// query tiles that can see those keys.  Per query tile, five tensor-core products:
//   S  = Q K^T          dP = dO V^T                       (into TMEM, rows = queries)
//   dV += P^T dO        dK += dS^T Q                      (accumulate in TMEM across the whole loop, rows = keys)
//   dQ  = dS K                                            (TMEM -> shared staging -> fp32 reduction into dq_acc)
// with P = exp2(S*c - lse) and dS = scale * P * (dP - delta) computed in between and written to shared memory in a
// layout that serves both as a K-major operand (dS K) and, transposed, as an MN-major operand (P^T dO, dS^T Q).
//   warps 0-7  two compute warpgroups: thread = one query row x one half (64 keys) of the S / dP tiles.  A thread pulls
//              its 64 scores and 64 dP values from TMEM in one go and hands the columns straight back, so the tensor core
//              computes S / dP of the next query tile while P / dS of this one are formed; it then drains its quarter
//              of the previous tile's dQ (TMEM -> shared staging -> fp32 reduction into dq_acc)
//   warp 8     TMA producer      warp 9     MMA issuer      (warps 10-11 only take part in the register hand-over)
#include <cuda_bf16.h>

#include "common/host.h"
#include "common/ptx.cuh"

namespace dptb {

struct AttnBwdParams {
  const float* lse;      // [B, Hq, Sq] natural log
  const float* delta;    // [B, Hq, Sq] rowsum(dO * O)
  float* dq_acc;         // [B*Sq, Hq*64] fp32, zero-initialised
  __nv_bfloat16* dk;     // [B*Sk, lddk]
  __nv_bfloat16* dv;
  long long lddk, lddv;
  int B, Sq, Sk, Hq, Hkv;
  int causal, q_offset;
  float scale, scale_log2;
};

__device__ __forceinline__ float fast_exp2_b(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Opt-in phase timers (compile with -DDPTB_ATTN_PROFILE), SM clock cycles summed over all CTAs:
//   compute thread 0:  [0] wait S/dP  [1] TMEM -> registers  [2] P / dS math  [3] wait for the previous products
//                      [4] stores + signal  [5] dQ drain  [6] loop total  [7] iterations
//   MMA issuer:        [8] wait Q/dO  [9] wait S/dP drained  [10] wait P/dS  [11] wait dQ drained  [12] loop total
#ifdef DPTB_ATTN_PROFILE
__device__ unsigned long long g_attn_bwd_prof[16];
#define BWD_PROF_MARK(t) const long long t = clock64()
#define BWD_PROF_ADD(slot, t0, t1) prof_acc[slot] += (t1) - (t0)
#else
#define BWD_PROF_MARK(t)
#define BWD_PROF_ADD(slot, t0, t1)
#endif

constexpr int kBwdHD = 64;
constexpr int kBwdTile = 128;
constexpr int kBwdThreads = 384;
// Registers per thread after the hand-over (the CTA starts with 384 x 168 and the pool does not grow).
constexpr int kBwdComputeRegs = 216;
constexpr int kBwdProducerRegs = 72;
static_assert(2 * 128 * kBwdComputeRegs + 128 * kBwdProducerRegs <= kBwdThreads * 168, "register hand-over must balance");
constexpr int kBwdStages = 2;
constexpr int kDqStride = 68;  // floats per staged dQ row (padding keeps 16-byte accesses conflict-free)

struct AttnBwdSmem {
  static constexpr int kTileBytes = kBwdTile * kBwdHD * 2;       // 16 KB: one [128 x 64] bf16 tile
  static constexpr int kPBytes = kBwdTile * kBwdTile * 2;        // 32 KB
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kKOff + kTileBytes;
  static constexpr int kQOff = kVOff + kTileBytes;               // [stages]
  static constexpr int kDOOff = kQOff + kBwdStages * kTileBytes; // [stages]
  static constexpr int kPOff = kDOOff + kBwdStages * kTileBytes;
  static constexpr int kDSOff = kPOff + kPBytes;
  static constexpr int kDqOff = kDSOff + kPBytes;
  static constexpr int kDqBytes = kBwdTile * kDqStride * 4;
  static constexpr int kBarOff = kDqOff + kDqBytes;
  static constexpr int kNumBars = 1 + 2 * kBwdStages + 7;
  static constexpr int kTotal = kBarOff + kNumBars * 8 + 16 + 1024;
};

__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                const AttnBwdParams p) {
  using L = AttnBwdSmem;
  constexpr int HD = kBwdHD;
  constexpr int TMEM_COLS = 512;
  constexpr int kSCol = 0, kDPCol = 128, kDVCol = 256, kDKCol = 320, kDQCol = 384;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = kv_full + 1;               // [stages]
  uint64_t* qdo_empty = qdo_full + kBwdStages;    // [stages]
  uint64_t* sdp_full = qdo_empty + kBwdStages;    // S and dP of the current query tile are in TMEM
  uint64_t* sdp_empty = sdp_full + 1;             // ... and have been copied to registers by all 256 compute threads
  uint64_t* pds_full = sdp_empty + 1;             // P and dS are in shared memory
  uint64_t* dq_full = pds_full + 1;
  uint64_t* dq_empty = dq_full + 1;
  uint64_t* dkv_full = dq_empty + 1;
  uint64_t* drain_bar = dkv_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, kv_head = blockIdx.y, batch = blockIdx.z;
  const int key0 = kt * kBwdTile;
  const int group = p.Hq / p.Hkv;
  const int n_q_tiles = (p.Sq + kBwdTile - 1) / kBwdTile;
  // First query tile with a row that can see key0 (causal: i + q_offset >= key0).
  int i_start = 0;
  if (p.causal) {
    const int first_row = key0 - p.q_offset;
    i_start = first_row > 0 ? first_row / kBwdTile : 0;
  }
  const int tiles_per_head = n_q_tiles > i_start ? n_q_tiles - i_start : 0;
  const int total_iters = tiles_per_head * group;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 9) {
    if (lane == 0) {
      mbar_init(kv_full, 1);
      for (int s = 0; s < kBwdStages; ++s) {
        mbar_init(&qdo_full[s], 1);
        mbar_init(&qdo_empty[s], 1);
      }
      mbar_init(sdp_full, 1);
      mbar_init(sdp_empty, 2 * kBwdTile);
      mbar_init(pds_full, 2 * kBwdTile);
      mbar_init(dq_full, 1);
      mbar_init(dq_empty, 2 * kBwdTile);
      mbar_init(dkv_full, 1);
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

  if (warp >= 8) {
    warpgroup_reg_dec<kBwdProducerRegs>();
  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && total_iters > 0) {
      mbar_arrive_expect_tx(kv_full, 2 * L::kTileBytes);
      tma_load_3d(smem + L::kKOff, &tmK, kv_full, kv_head * HD, key0, batch);
      tma_load_3d(smem + L::kVOff, &tmV, kv_full, kv_head * HD, key0, batch);
      int it = 0;
      for (int g = 0; g < group && !*abort_flag; ++g) {
        const int head = kv_head * group + g;
        for (int i = i_start; i < n_q_tiles; ++i, ++it) {
          const int s = it % kBwdStages;
          const uint32_t ph = (it / kBwdStages) & 1;
          if (!mbar_wait(&qdo_empty[s], ph ^ 1, abort_flag, kWaitEmptyTimeout)) break;
          mbar_arrive_expect_tx(&qdo_full[s], 2 * L::kTileBytes);
          tma_load_3d(smem + L::kQOff + s * L::kTileBytes, &tmQ, &qdo_full[s], head * HD, i * kBwdTile, batch);
          tma_load_3d(smem + L::kDOOff + s * L::kTileBytes, &tmDO, &qdo_full[s], head * HD, i * kBwdTile, batch);
        }
      }
      if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(kv_full, 0) && global_timer_ns() - t0 < kWaitLimitNs / 4) {}
        for (int j = max(0, it - kBwdStages); j < it; ++j)
          while (!mbar_try_wait(&qdo_full[j % kBwdStages], (j / kBwdStages) & 1) &&
                 global_timer_ns() - t0 < kWaitLimitNs / 4) {}
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && total_iters > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kBwdTile, kBwdTile, false, false);   // S, dP
      constexpr uint32_t idesc_kv = make_idesc_bf16(kBwdTile, HD, true, true);          // dV, dK
      constexpr uint32_t idesc_q = make_idesc_bf16(kBwdTile, HD, false, true);          // dQ
      const uint32_t k_addr = smem_u32(smem + L::kKOff), v_addr = smem_u32(smem + L::kVOff);
      const uint32_t p_addr = smem_u32(smem + L::kPOff), ds_addr = smem_u32(smem + L::kDSOff);
      bool ok = mbar_wait(kv_full, 0, abort_flag, kWaitFullTimeout);
      bool issued_any = false;
      // S = Q K^T and dP = dO V^T of query tile `it` (operands in stage it % stages).
      auto issue_sdp = [&](int it) {
        const int s = it % kBwdStages;
        const uint32_t q_addr = smem_u32(smem + L::kQOff + s * L::kTileBytes);
        const uint32_t do_addr = smem_u32(smem + L::kDOOff + s * L::kTileBytes);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          umma_bf16(tmem_base + kSCol, make_smem_desc(q_addr + kk * 32, 16, 1024),
                    make_smem_desc(k_addr + kk * 32, 16, 1024), idesc_s, kk != 0);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          umma_bf16(tmem_base + kDPCol, make_smem_desc(do_addr + kk * 32, 16, 1024),
                    make_smem_desc(v_addr + kk * 32, 16, 1024), idesc_s, kk != 0);
        umma_commit(sdp_full);
        issued_any = true;
      };
      if (ok) ok = mbar_wait(&qdo_full[0], 0, abort_flag, kWaitFullTimeout);
      if (ok) {
        tc_fence_after_sync();
        issue_sdp(0);
      }
#ifdef DPTB_ATTN_PROFILE
      long long prof_acc[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
      const long long prof_begin = clock64();
#endif
      for (int it = 0; it < total_iters && ok; ++it) {
        const int s = it % kBwdStages;
        const uint32_t q_addr = smem_u32(smem + L::kQOff + s * L::kTileBytes);
        const uint32_t do_addr = smem_u32(smem + L::kDOOff + s * L::kTileBytes);
        // (a) S / dP of the next query tile, as soon as the compute warps have copied this tile's out of TMEM.
        if (it + 1 < total_iters) {
          const int s1 = (it + 1) % kBwdStages;
          BWD_PROF_MARK(m0);
          ok = mbar_wait(&qdo_full[s1], ((it + 1) / kBwdStages) & 1, abort_flag, kWaitFullTimeout);
          BWD_PROF_MARK(m1);
          if (ok) ok = mbar_wait(sdp_empty, it & 1, abort_flag, kWaitTmemEmptyTimeout);
          BWD_PROF_MARK(m2);
          BWD_PROF_ADD(8, m0, m1);
          BWD_PROF_ADD(9, m1, m2);
          if (!ok) break;
          tc_fence_after_sync();
          issue_sdp(it + 1);
        }
        // (b) the three products that consume P / dS of this tile.
        BWD_PROF_MARK(m3);
        ok = mbar_wait(pds_full, it & 1, abort_flag, kWaitFlagTimeout);
        BWD_PROF_MARK(m4);
        BWD_PROF_ADD(10, m3, m4);
        if (!ok) break;
        tc_fence_after_sync();
        // dV += P^T dO ; dK += dS^T Q    (A: [q rows][keys] read as MN-major, B: [q rows][hd] read as MN-major)
#pragma unroll
        for (int kk = 0; kk < kBwdTile / 16; ++kk)
          umma_bf16(tmem_base + kDVCol, make_smem_desc(p_addr + kk * 2048, kBwdTile * 128, 1024),
                    make_smem_desc(do_addr + kk * 2048, kBwdTile * 128, 1024), idesc_kv, (it | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < kBwdTile / 16; ++kk)
          umma_bf16(tmem_base + kDKCol, make_smem_desc(ds_addr + kk * 2048, kBwdTile * 128, 1024),
                    make_smem_desc(q_addr + kk * 2048, kBwdTile * 128, 1024), idesc_kv, (it | kk) != 0);
        if (it > 0) {
          BWD_PROF_MARK(m5);
          ok = mbar_wait(dq_empty, (it - 1) & 1, abort_flag, kWaitFlagTimeout);
          BWD_PROF_MARK(m6);
          BWD_PROF_ADD(11, m5, m6);
          if (!ok) break;
          tc_fence_after_sync();
        }
        // dQ = dS K   (A: dS K-major over keys, B: K tile [keys][hd] read as MN-major)
#pragma unroll
        for (int kk = 0; kk < kBwdTile / 16; ++kk)
          umma_bf16(tmem_base + kDQCol,
                    make_smem_desc(ds_addr + (kk / 4) * (kBwdTile * 128) + (kk % 4) * 32, 16, 1024),
                    make_smem_desc(k_addr + kk * 2048, kBwdTile * 128, 1024), idesc_q, kk != 0);
        umma_commit(dq_full);
        umma_commit(&qdo_empty[s]);
        issued_any = true;
      }
#ifdef DPTB_ATTN_PROFILE
      prof_acc[12] = clock64() - prof_begin;
      for (int i = 8; i < 13; ++i) atomicAdd(&g_attn_bwd_prof[i], (unsigned long long)prof_acc[i]);
#endif
      if (ok) umma_commit(dkv_full);
      if (*abort_flag && issued_any) {
        umma_commit(drain_bar);
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < kWaitLimitNs / 4) {}
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    warpgroup_reg_inc<kBwdComputeRegs>();
    const int q = warp & 3;          // TMEM lane quarter
    const int half = warp >> 2;      // which 64 keys of the tile (and which 32 columns of dQ) this thread handles
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    uint8_t* p_tile = smem + L::kPOff + half * (kBwdTile * 128);     // 64-key block `half` of the K-major tiles
    uint8_t* ds_tile = smem + L::kDSOff + half * (kBwdTile * 128);
    float* dq_stage = reinterpret_cast<float*>(smem + L::kDqOff);
    bool ok = true;

    // Drains this thread's part of dQ of iteration `itp` (head hp, query tile ip): TMEM -> staging -> fp32 reduction.
    // Its phase of dq_full has been waited for by the caller.
    auto flush_dq = [&](int hp, int ip) {
      tc_fence_after_sync();
      uint32_t r[32];
      tmem_ld_32x32(lane_addr + kDQCol + half * 32, r);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(dq_empty);
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<float4*>(dq_stage + row * kDqStride + half * 32 + i) =
            make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                        __uint_as_float(r[i + 3]));
      __syncwarp();
      // This warp staged rows [q*32, q*32+32) x columns [half*32, half*32+32) and reduces exactly that block:
      // 4 rows of 128 bytes per instruction.
#pragma unroll
      for (int rr = 0; rr < 32; rr += 4) {
        const int r_loc = q * 32 + rr + (lane >> 3);
        const int col = half * 32 + (lane & 7) * 4;
        const int qi = ip * kBwdTile + r_loc;
        if (qi < p.Sq) {
          const float4 v = *reinterpret_cast<const float4*>(dq_stage + r_loc * kDqStride + col);
          float* dst = p.dq_acc + ((long long)batch * p.Sq + qi) * ((long long)p.Hq * HD) + (long long)hp * HD + col;
          red_add_v4(dst, v.x, v.y, v.z, v.w);
        }
      }
      __syncwarp();
    };

    int it = 0;
    int prev_h = 0, prev_i = 0;
#ifdef DPTB_ATTN_PROFILE
    long long prof_acc[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    const long long prof_begin = clock64();
#endif
    for (int g = 0; g < group && ok; ++g) {
      const int head = kv_head * group + g;
      for (int i = i_start; i < n_q_tiles && ok; ++i, ++it) {
        const int qi = i * kBwdTile + row;
        const bool row_ok = qi < p.Sq;
        const long long stat = ((long long)batch * p.Hq + head) * p.Sq + (row_ok ? qi : 0);
        const float lse_nat = row_ok ? p.lse[stat] : 0.0f;
        const float delta = row_ok ? p.delta[stat] : 0.0f;
        const bool dead = !row_ok || lse_nat == -INFINITY;
        const float lse2 = dead ? INFINITY : lse_nat * 1.4426950408889634f;   // dead rows: exp2(-inf) = 0
        const int key_limit = p.causal ? min(p.Sk - 1, qi + p.q_offset) : p.Sk - 1;
        const int kbase = key0 + half * 64;
        BWD_PROF_MARK(c0);
        ok = __all_sync(0xffffffffu, mbar_wait(sdp_full, it & 1, abort_flag, kWaitTmemFullTimeout));
        if (!ok) break;
        BWD_PROF_MARK(c1);
        tc_fence_after_sync();
        uint32_t rs[64], rp[64];
        tmem_ld_32x32(lane_addr + kSCol + half * 64, reinterpret_cast<uint32_t(&)[32]>(rs[0]));
        tmem_ld_32x32(lane_addr + kSCol + half * 64 + 32, reinterpret_cast<uint32_t(&)[32]>(rs[32]));
        tmem_ld_32x32(lane_addr + kDPCol + half * 64, reinterpret_cast<uint32_t(&)[32]>(rp[0]));
        tmem_ld_32x32(lane_addr + kDPCol + half * 64 + 32, reinterpret_cast<uint32_t(&)[32]>(rp[32]));
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive(sdp_empty);   // the tensor core may overwrite S / dP with the next query tile's
        BWD_PROF_MARK(c2);
        uint32_t pk_p[32], pk_ds[32];
        const bool need_mask = kbase + 63 > key_limit;
#pragma unroll
        for (int e = 0; e < 64; e += 2) {
          float p0 = fast_exp2_b(fmaf(__uint_as_float(rs[e]), p.scale_log2, -lse2));
          float p1 = fast_exp2_b(fmaf(__uint_as_float(rs[e + 1]), p.scale_log2, -lse2));
          if (need_mask) {
            if (kbase + e > key_limit) p0 = 0.0f;
            if (kbase + e + 1 > key_limit) p1 = 0.0f;
          }
          const float d0 = p0 * (__uint_as_float(rp[e]) - delta) * p.scale;
          const float d1 = p1 * (__uint_as_float(rp[e + 1]) - delta) * p.scale;
          pk_p[e >> 1] = pack_bf16x2(p0, p1);
          pk_ds[e >> 1] = pack_bf16x2(d0, d1);
        }
        BWD_PROF_MARK(c3);
        // P / dS of the previous iteration must have been consumed before they are overwritten: every MMA of that
        // iteration has completed once its dq_full phase has.
        if (it > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(dq_full, (it - 1) & 1, abort_flag, kWaitTmemFullTimeout));
          if (!ok) break;
        }
        BWD_PROF_MARK(c4);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int off = row * 128 + (int)(((uint32_t)e ^ (uint32_t)(row & 7)) << 4);
          *reinterpret_cast<uint4*>(p_tile + off) = make_uint4(pk_p[e * 4], pk_p[e * 4 + 1], pk_p[e * 4 + 2], pk_p[e * 4 + 3]);
          *reinterpret_cast<uint4*>(ds_tile + off) = make_uint4(pk_ds[e * 4], pk_ds[e * 4 + 1], pk_ds[e * 4 + 2], pk_ds[e * 4 + 3]);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(pds_full);
        BWD_PROF_MARK(c5);
        if (it > 0) flush_dq(prev_h, prev_i);
        BWD_PROF_MARK(c6);
        BWD_PROF_ADD(0, c0, c1);
        BWD_PROF_ADD(1, c1, c2);
        BWD_PROF_ADD(2, c2, c3);
        BWD_PROF_ADD(3, c3, c4);
        BWD_PROF_ADD(4, c4, c5);
        BWD_PROF_ADD(5, c5, c6);
        prev_h = head;
        prev_i = i;
      }
    }
#ifdef DPTB_ATTN_PROFILE
    if (threadIdx.x == 0) {
      prof_acc[6] = clock64() - prof_begin;
      prof_acc[7] = it;
      for (int i = 0; i < 8; ++i) atomicAdd(&g_attn_bwd_prof[i], (unsigned long long)prof_acc[i]);
    }
#endif
    if (ok && total_iters > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(dq_full, (total_iters - 1) & 1, abort_flag, kWaitTmemFullTimeout));
      if (ok) flush_dq(prev_h, prev_i);
    }

    // dK / dV of this key tile.
    const int key = key0 + row;
    if (total_iters == 0) {
      if (key < p.Sk) {
        __nv_bfloat16* dkp = p.dk + ((long long)batch * p.Sk + key) * p.lddk + (long long)kv_head * HD;
        __nv_bfloat16* dvp = p.dv + ((long long)batch * p.Sk + key) * p.lddv + (long long)kv_head * HD;
        for (int d = half * 32; d < half * 32 + 32; d += 8) {
          *reinterpret_cast<uint4*>(dkp + d) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(dvp + d) = make_uint4(0, 0, 0, 0);
        }
      }
    } else if (ok && __all_sync(0xffffffffu, mbar_wait(dkv_full, 0, abort_flag, kWaitTmemFullTimeout))) {
      tc_fence_after_sync();
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* base = which == 0 ? p.dv : p.dk;
        const long long ld = which == 0 ? p.lddv : p.lddk;
        const uint32_t col0 = which == 0 ? kDVCol : kDKCol;
        {
          const int c = half;   // each compute warpgroup writes 32 of the 64 columns
          uint32_t r[32];
          tmem_ld_32x32(lane_addr + col0 + c * 32, r);
          tmem_ld_wait();
          if (key < p.Sk) {
            __nv_bfloat16* dst = base + ((long long)batch * p.Sk + key) * ld + (long long)kv_head * HD + c * 32;
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(r[e]), __uint_as_float(r[e + 1]));
              u.y = pack_bf16x2(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
              u.z = pack_bf16x2(__uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
              u.w = pack_bf16x2(__uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
              *reinterpret_cast<uint4*>(dst + e) = u;
            }
          }
        }
      }
      tc_fence_before_sync();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

// delta[b, h, s] = sum_d dO * O over one head row of 64 values: 8 lanes per (token, head), 16 bytes per lane, so a
// warp reads four consecutive heads of a token as one 512-byte run.
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long ldo, const __nv_bfloat16* __restrict__ dout,
                  long long lddo, float* __restrict__ delta, int B, int S, int H, int hd) {
  const int sub = threadIdx.x & 7;
  const long long total = (long long)B * S * H;
  for (long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3; w < total;
       w += ((long long)gridDim.x * blockDim.x) >> 3) {
    const int h = (int)(w % H);
    const long long tok = w / H;  // b*S + s
    const uint4 a = *reinterpret_cast<const uint4*>(o + tok * ldo + (long long)h * hd + sub * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(dout + tok * lddo + (long long)h * hd + sub * 8);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
    float acc = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x +
                a3.y * b3.y;
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    if (sub == 0) {
      const long long bb = tok / S, ss = tok % S;
      delta[(bb * H + h) * S + ss] = acc;
    }
  }
}

// dq[r, c] = bf16(dq_acc[r, c])
__global__ void __launch_bounds__(256)
attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long lddq, long long rows,
                       int cols) {
  const long long n4 = rows * (cols / 4);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (cols / 4);
    const int c = (int)(i % (cols / 4)) * 4;
    const float4 v = *reinterpret_cast<const float4*>(acc + r * cols + c);
    uint2 u;
    u.x = pack_bf16x2(v.x, v.y);
    u.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dq + r * lddq + c) = u;
  }
}

static int encode_tmap_seq_b(CUtensorMap* map, const void* base, int heads, int hd, int seq, int batch, long long ld) {
  const uint64_t dims[3] = {(uint64_t)heads * hd, (uint64_t)seq, (uint64_t)batch};
  const uint64_t strides[2] = {(uint64_t)ld * 2, (uint64_t)seq * ld * 2};
  const uint32_t box[3] = {64, (uint32_t)kBwdTile, 1};
  return encode_tmap_nd_bf16(map, base, 3, dims, strides, box);
}

}  // namespace dptb

using namespace dptb;

struct DptbAttnBwdArgs {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* dout;
  const float* lse;
  float* delta;    // [B, Hq, Sq] scratch, written here
  float* dq_acc;   // [B*Sq, Hq*hd] fp32 scratch, zeroed by the caller
  void* dq;
  void* dk;
  void* dv;
  long long ldq, ldk, ldv, ldo, lddo, lddq, lddk, lddv;
  int B, Sq, Sk, Hq, Hkv, head_dim;
  int causal, q_offset;
  float scale;
};

// Phase timers (see DPTB_ATTN_PROFILE): copies the 16 counters out and zeroes them; -5 when not compiled in.
extern "C" int dptb_attn_bwd_profile_read(unsigned long long* out) {
#ifdef DPTB_ATTN_PROFILE
  int rc = (int)cudaMemcpyFromSymbol(out, g_attn_bwd_prof, sizeof(unsigned long long) * 16);
  if (rc) return rc;
  static unsigned long long zeros[16];
  return (int)cudaMemcpyToSymbol(g_attn_bwd_prof, zeros, sizeof(zeros));
#else
  (void)out;
  return kErrUnsupported;
#endif
}

extern "C" int dptb_attn_bwd(const DptbAttnBwdArgs* a, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  if (a->B <= 0 || a->Sq <= 0 || a->Hq <= 0) return 0;
  if (a->head_dim != kBwdHD) return kErrUnsupported;
  if (a->Sk <= 0 || a->Hkv <= 0 || a->Hq % a->Hkv) return kErrBadShape;
  if ((a->ldq % 8) || (a->ldk % 8) || (a->ldv % 8) || (a->ldo % 8) || (a->lddo % 8) || (a->lddq % 8) ||
      (a->lddk % 8) || (a->lddv % 8))
    return kErrBadShape;
  if (((reinterpret_cast<uintptr_t>(a->dq) | reinterpret_cast<uintptr_t>(a->dk) | reinterpret_cast<uintptr_t>(a->dv) |
        reinterpret_cast<uintptr_t>(a->dq_acc)) & 15) != 0)
    return kErrBadShape;
  using L = AttnBwdSmem;
  const long long groups = (long long)a->B * a->Sq * a->Hq;   // 8 lanes each, 32 groups per block
  int dgrid = (int)((groups + 31) / 32);
  if (dgrid > sm_count() * 16) dgrid = sm_count() * 16;
  attn_delta_kernel<<<dgrid, 256, 0, st>>>((const __nv_bfloat16*)a->o, a->ldo, (const __nv_bfloat16*)a->dout, a->lddo,
                                          a->delta, a->B, a->Sq, a->Hq, kBwdHD);
  DPTB_CUDA_OK(cudaGetLastError());

  CUtensorMap tmQ, tmK, tmV, tmDO;
  int rc = encode_tmap_seq_b(&tmQ, a->q, a->Hq, kBwdHD, a->Sq, a->B, a->ldq);
  if (rc) return rc;
  rc = encode_tmap_seq_b(&tmK, a->k, a->Hkv, kBwdHD, a->Sk, a->B, a->ldk);
  if (rc) return rc;
  rc = encode_tmap_seq_b(&tmV, a->v, a->Hkv, kBwdHD, a->Sk, a->B, a->ldv);
  if (rc) return rc;
  rc = encode_tmap_seq_b(&tmDO, a->dout, a->Hq, kBwdHD, a->Sq, a->B, a->lddo);
  if (rc) return rc;
  AttnBwdParams p;
  p.lse = a->lse; p.delta = a->delta; p.dq_acc = a->dq_acc;
  p.dk = static_cast<__nv_bfloat16*>(a->dk); p.dv = static_cast<__nv_bfloat16*>(a->dv);
  p.lddk = a->lddk; p.lddv = a->lddv;
  p.B = a->B; p.Sq = a->Sq; p.Sk = a->Sk; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.causal = a->causal; p.q_offset = a->q_offset;
  p.scale = a->scale;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  DPTB_CUDA_OK(cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
  dim3 grid((a->Sk + kBwdTile - 1) / kBwdTile, a->Hkv, a->B);
  attn_bwd_kernel<<<grid, kBwdThreads, L::kTotal, st>>>(tmQ, tmK, tmV, tmDO, p);
  DPTB_CUDA_OK(cudaGetLastError());
  const long long rows = (long long)a->B * a->Sq;
  const int cols = a->Hq * kBwdHD;
  long long cgrid = (rows * (cols / 4) + 255) / 256;
  if (cgrid > sm_count() * 16) cgrid = sm_count() * 16;
  attn_dq_convert_kernel<<<(int)cgrid, 256, 0, st>>>(a->dq_acc, static_cast<__nv_bfloat16*>(a->dq), a->lddq, rows, cols);
  return counted(3, (int)cudaGetLastError());
}
