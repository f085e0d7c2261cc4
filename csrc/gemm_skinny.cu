// Skinny GEMM for decode-sized inputs:  out[M, N] = x[M, K] @ W[N, K]^T  with M <= 64 rows (one new token per
// sequence), W an nn.Linear weight.  The reference runs such products through the same tiled kernel as everything else
// (lib/native/src/kernels/matmul.cuh:27-63); at M = 32 the work is streaming W from HBM once, and what decides the
// speed is how many bytes are in flight: a tile-per-CTA GEMM with 128-row tiles puts only N / 128 CTAs on the machine.
//
// Here the operands are swapped on the tensor core: a CTA owns 128 rows of W (the M = 128 side of tcgen05.mma, all
// useful bytes) and one slice of K; x is the narrow N = 32 / 64 side.  Work units = (N / 128) x (K splits) are chosen
// to fill the SMs once, each with an 8-stage TMA ring (128 KB of W in flight per SM).  D[128 weight rows, M] lands
// in 32 / 64 TMEM columns; a thread of the four epilogue warps owns one weight row = one output column.
//   splits == 1: the epilogue writes out[m, n] directly (lanes = consecutive n, so stores coalesce);
//   splits  > 1: fp32 partials go to a workspace, the last unit of a tile (per-tile counter) sums them in split order
//                (deterministic) and runs the epilogue.
// Row-parallel Linear of a tensor-parallel group (all-reduce over ranks, + bias, + residual) is fused the same way as
// in the big GEMM: the finished local tile goes to this rank's symmetric partial buffer, the tile's owner rank is
// flagged, the owner reduces over the ranks (multimem.ld_reduce through the NVSwitch, else peer loads) and writes the
// result into every rank's output (multimem.st, else peer stores); the last CTA runs the end-of-kernel handshake.
#include <cuda_bf16.h>

#include "common/gemm_args.h"
#include "common/host.h"
#include "common/peer.cuh"
#include "common/ptx.cuh"

namespace dptb {

// Opt-in timeline (compile with -DDPTB_SKINNY_PROFILE): globaltimer stamps (ns) of work unit 0 and of the last unit of
// tile 0: [0] kernel entry  [1] barriers + TMEM ready  [2] first stage landed  [3] accumulator complete
// [4] partials written  [5] tile counter known  [6] splits folded  [7] output written
#ifdef DPTB_SKINNY_PROFILE
__device__ unsigned long long g_skinny_prof[8];
#define SK_STAMP(slot, cond) do { if (cond) g_skinny_prof[slot] = global_timer_ns(); } while (0)
#else
#define SK_STAMP(slot, cond)
#endif

constexpr int kSkBM = 128;       // weight rows per CTA
constexpr int kSkBK = 64;
constexpr int kSkStages = 8;
constexpr int kSkThreads = 192;  // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue

struct SkinnyAr {
  int world, rank, use_nvls;
  __nv_bfloat16* partial;
  const __nv_bfloat16* peer_partial[kMaxRanks];
  const __nv_bfloat16* mc_partial;
  __nv_bfloat16* out_peer[kMaxRanks];
  __nv_bfloat16* mc_out;
  uint32_t* flags_peer[kMaxRanks];
  int max_tiles;
  uint32_t* epoch;
  unsigned int* exit_counter;
};

// One-shot all-reduce for these small outputs (a few hundred KB per rank): every rank stores the fp32 tile it finished
// into slot [parity][its rank][tile] of EVERY rank's symmetric slot buffer, each value as one 8-byte word {fp32 bits,
// launch number} (a single-copy-atomic store, so a word that shows the launch number also shows the value); a rank
// then polls the slots of all ranks in its OWN memory and sums them in rank order.  One NVLink hop instead of gather +
// broadcast, no fence, no flag, no end-of-kernel handshake.  Slots alternate between two halves by launch parity: a
// rank finishes launch e - 1 only after it has received all tiles of e - 1 from every rank, so every rank has started
// e - 1 and hence finished reading the slots of e - 2 before anyone overwrites them in launch e.
struct SkinnyOneShot {
  int world, rank;
  uint2* slots_local;                 // [2][kMaxRanks][max_tiles][64][128] words
  uint2* slots_peer[kMaxRanks];
  int max_tiles;
  uint32_t* epoch;                    // local launch counter
  unsigned int* exit_counter;         // local, zero between launches
};

struct SkinnyParams {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* bias;        // [N] bf16 or null
  const __nv_bfloat16* residual;    // [M, ldr] or null
  long long ldr;
  int num_kb, splits, kb_per_split;
  int vec_out;                      // C / residual 16-byte aligned, leading dimensions and N multiples of 8
  float* ws;                        // [tile][split][MP][128] fp32
  int* counters;                    // per tile, zero between launches
  SkinnyAr ar;
  SkinnyOneShot os;
};

// 8-byte words of the flag-in-data protocol: one single-copy-atomic access each, at system scope.
__device__ __forceinline__ void st_relaxed_sys_v2(uint2* p, uint32_t a, uint32_t b) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_relaxed_sys_v2(const uint2* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_v4(uint2* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const uint2* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <int MP>
struct SkinnySmem {
  static constexpr int kWBytes = kSkBM * kSkBK * 2;     // 16 KB
  static constexpr int kXBytes = MP * kSkBK * 2;        // 4 / 8 KB
  static constexpr int kStage = kWBytes + kXBytes;
  static constexpr int kBarOff = kSkStages * kStage;
  static constexpr int kTotal = kBarOff + (2 * kSkStages + 2) * 8 + 64 + 1024;
};

// Final values of one tile -> output (non-tensor-parallel): thread = output column n, v[m] over the rows.
template <int MP>
__device__ __forceinline__ void skinny_store(const SkinnyParams& p, int n, const float (&v)[MP]) {
  if (n >= p.N) return;
  const float b = p.bias ? __bfloat162float(p.bias[n]) : 0.0f;
#pragma unroll
  for (int m = 0; m < MP; ++m) {
    if (m < p.M) {
      float o = v[m] + b;
      if (p.residual) o += __bfloat162float(p.residual[(long long)m * p.ldr + n]);
      p.C[(long long)m * p.ldc + n] = __float2bfloat16(o);
    }
  }
}

template <int MP>
__global__ void __launch_bounds__(kSkThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const SkinnyParams p) {
  using L = SkinnySmem<MP>;
  constexpr int TMEM_COLS = MP < 32 ? 32 : MP;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + kSkStages;
  uint64_t* acc_full = empty_bar + kSkStages;
  uint64_t* drain_bar = acc_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* epi_ctr = reinterpret_cast<int*>(tmem_slot + 2);
  volatile int* epi_last = reinterpret_cast<volatile int*>(tmem_slot + 3);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / p.splits;
  const int split = blockIdx.x % p.splits;
  const int n0 = tile * kSkBM;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
  const uint32_t ar_epoch = p.ar.world > 0 ? *reinterpret_cast<volatile uint32_t*>(p.ar.epoch) + 1u : 0u;
  const uint32_t os_epoch = p.os.world > 0 ? *reinterpret_cast<volatile uint32_t*>(p.os.epoch) + 1u : 0u;

  SK_STAMP(0, blockIdx.x == 0 && threadIdx.x == 0);
  pdl_launch_dependents();   // the small kernel after this one waits for this grid's completion at its own top
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *epi_ctr = 0;
    *epi_last = 0;
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    if (lane == 0) {
      for (int s = 0; s < kSkStages; ++s) {
        mbar_init(&full_bar[s], 1);
        mbar_init(&empty_bar[s], 1);
      }
      mbar_init(acc_full, 1);
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
  SK_STAMP(1, blockIdx.x == 0 && threadIdx.x == 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // The weights do not depend on the kernel before this one: the first ring-full of weight tiles is requested at
      // once, then (programmatic dependent launch) the predecessor's completion is awaited, then the activation
      // tiles of those stages follow.  Every stage's barrier expects both tiles.
      const int pre = max(0, min(kb1 - kb0, kSkStages));
      for (int i = 0; i < pre; ++i) {
        mbar_arrive_expect_tx(&full_bar[i], L::kStage);
        tma_load_2d(smem + i * L::kStage, &tmW, &full_bar[i], (kb0 + i) * kSkBK, n0);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d(smem + i * L::kStage + L::kWBytes, &tmX, &full_bar[i], (kb0 + i) * kSkBK, 0);
      int issued = pre;
      for (int kb = kb0 + pre; kb < kb1; ++kb, ++issued) {
        const int s = issued % kSkStages;
        const uint32_t ph = (issued / kSkStages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, kWaitEmptyTimeout)) break;
        mbar_arrive_expect_tx(&full_bar[s], L::kStage);
        uint8_t* w_dst = smem + s * L::kStage;
        tma_load_2d(w_dst, &tmW, &full_bar[s], kb * kSkBK, n0);
        tma_load_2d(w_dst + L::kWBytes, &tmX, &full_bar[s], kb * kSkBK, 0);
      }
      if (*abort_flag) {
        // Do not leave while a tile copy may still be writing this CTA's shared memory.
        const int n = issued < kSkStages ? issued : kSkStages;
        const uint64_t t0 = global_timer_ns();
        for (int j = 0; j < n; ++j) {
          const int i = issued - 1 - j;
          while (!mbar_try_wait(&full_bar[i % kSkStages], (i / kSkStages) & 1) &&
                 global_timer_ns() - t0 < kWaitLimitNs / 4) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kSkBM, MP, false, false);
      bool issued_any = false, ok = true;
      int consumed = 0;
      for (int kb = kb0; kb < kb1; ++kb, ++consumed) {
        const int s = consumed % kSkStages;
        const uint32_t ph = (consumed / kSkStages) & 1;
        if (!mbar_wait(&full_bar[s], ph, abort_flag, kWaitFullTimeout)) { ok = false; break; }
        SK_STAMP(2, blockIdx.x == 0 && kb == kb0);
        tc_fence_after_sync();
        const uint32_t w_addr = smem_u32(smem + s * L::kStage);
        const uint32_t x_addr = w_addr + L::kWBytes;
#pragma unroll
        for (int k = 0; k < kSkBK / 16; ++k)
          umma_bf16(tmem_base, make_smem_desc(w_addr + k * 32, 16, 1024), make_smem_desc(x_addr + k * 32, 16, 1024),
                    idesc, (kb != kb0 || k != 0) ? 1u : 0u);
        issued_any = true;
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(acc_full);
      if (*abort_flag && issued_any) {
        umma_commit(drain_bar);
        const uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(drain_bar, 0) && global_timer_ns() - t0 < kWaitLimitNs / 4) {}
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (one TMEM lane quarter each)
    pdl_wait();   // nothing below may touch global memory before the predecessor has completed (an empty K range
                  // reaches the stores without passing through the producer's wait)
    const int q = warp & 3;
    const int n_local = q * 32 + lane;
    const int et = threadIdx.x - 64;           // 0..127 among the epilogue threads
    int epi_gen = 0;
    // Bounded barrier over the four epilogue warps.
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      epi_gen += 4;
      if (lane == 0) {
        __threadfence_block();
        atomicAdd(epi_ctr, 1);
        uint64_t t0 = 0;
        uint32_t spins = 0;
        while (*reinterpret_cast<volatile int*>(epi_ctr) < epi_gen) {
          if ((++spins & 0xff) == 0) {
            if (*abort_flag) break;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > kWaitLimitNs) {
              *abort_flag = 1;
              report_error(kWaitFlagTimeout);
              break;
            }
          }
        }
        __threadfence_block();
      }
      __syncwarp();
      return !*abort_flag;
    };
    bool ok = kb1 > kb0;
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0, abort_flag, kWaitTmemFullTimeout));
    SK_STAMP(3, blockIdx.x == 0 && et == 0);
    float v[MP];
#pragma unroll
    for (int m = 0; m < MP; ++m) v[m] = 0.0f;
    if (ok) {
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < MP / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[c * 32 + i] = __uint_as_float(r[i]);
      }
      tc_fence_before_sync();
    }
    bool have_tile = ok;   // this CTA holds the complete local sums of its tile in v
    if (ok && p.splits > 1) {
      float* mine = p.ws + ((size_t)tile * p.splits + split) * (MP * kSkBM);
#pragma unroll
      for (int m = 0; m < MP; ++m) mine[m * kSkBM + n_local] = v[m];
      __threadfence();
      ok = epi_sync();
      SK_STAMP(4, blockIdx.x == 0 && et == 0);
      if (ok && et == 0) {
        const int old = atomicAdd(&p.counters[tile], 1);
        const int last = old == p.splits - 1;
        if (last) p.counters[tile] = 0;   // ready for the next launch
        *epi_last = last;
      }
      if (ok) ok = epi_sync();
      have_tile = ok && *epi_last != 0;
      SK_STAMP(5, tile == 0 && have_tile && et == 0);
      if (have_tile) {
        __threadfence();
        const float* base = p.ws + (size_t)tile * p.splits * (MP * kSkBM) + n_local;
#pragma unroll
        for (int m = 0; m < MP; ++m) v[m] = 0.0f;
#pragma unroll 4
        for (int sp = 0; sp < p.splits; ++sp) {   // several splits' loads in flight; additions stay in split order
          const float* src = base + (size_t)sp * (MP * kSkBM);
#pragma unroll
          for (int m = 0; m < MP; ++m) v[m] += __ldcg(src + m * kSkBM);
        }
      }
    }
    SK_STAMP(6, tile == 0 && have_tile && et == 0);
    if (have_tile && p.ar.world == 0 && p.os.world == 0 && p.vec_out) {
      // Transpose through shared memory (the ring is idle by now) so that the output leaves as 16-byte vectors:
      // fp32 [MP][128] staging, then 16 lanes per output row.
      float* tile_s = reinterpret_cast<float*>(smem);
      const float b = (p.bias && n0 + n_local < p.N) ? __bfloat162float(p.bias[n0 + n_local]) : 0.0f;
#pragma unroll
      for (int m = 0; m < MP; ++m) tile_s[m * kSkBM + n_local] = v[m] + b;
      ok = epi_sync();
      const int cg = et & 15;
      const int col = n0 + cg * 8;
      if (ok && col < p.N) {
        for (int m = et >> 4; m < p.M; m += 8) {
          const float4 lo = *reinterpret_cast<const float4*>(tile_s + m * kSkBM + cg * 8);
          const float4 hi = *reinterpret_cast<const float4*>(tile_s + m * kSkBM + cg * 8 + 4);
          float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
          if (p.residual) {
            const uint4 r = *reinterpret_cast<const uint4*>(p.residual + (long long)m * p.ldr + col);
            const float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y), r2 = unpack_bf16x2(r.z), r3 = unpack_bf16x2(r.w);
            f[0] += r0.x; f[1] += r0.y; f[2] += r1.x; f[3] += r1.y;
            f[4] += r2.x; f[5] += r2.y; f[6] += r3.x; f[7] += r3.y;
          }
          uint4 o;
          o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
          o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
          *reinterpret_cast<uint4*>(p.C + (long long)m * p.ldc + col) = o;
        }
      }
      SK_STAMP(7, tile == 0 && et == 0);
    } else if (have_tile && p.ar.world == 0 && p.os.world == 0) {
      skinny_store<MP>(p, n0 + n_local, v);
    } else if (have_tile && p.os.world > 0) {
      // ---- one-shot all-reduce, flag-in-data: every value travels as one 8-byte store {fp32 bits, launch number}
      // into slot [parity][this rank][tile] of EVERY rank; a receiver polls the slots of all ranks in its own memory
      // until every word carries this launch's number and sums them in rank order.  No fence, no separate flag.
      const size_t tile_elems = (size_t)MP * kSkBM;
      const size_t rank_stride = (size_t)p.os.max_tiles * 64 * kSkBM;
      const size_t half_off = (size_t)(os_epoch & 1u) * kMaxRanks * rank_stride;
      float* tile_s = reinterpret_cast<float*>(smem);           // the ring is idle by now
#pragma unroll
      for (int m = 0; m < MP; ++m) tile_s[m * kSkBM + n_local] = v[m];
      ok = epi_sync();
      const int cg = et & 15;
      const int col = n0 + cg * 8;
      const size_t in_tile = (size_t)tile * tile_elems + cg * 8;
      if (ok) {
        const size_t mine = half_off + (size_t)p.os.rank * rank_stride + in_tile;
        for (int m = et >> 4; m < p.M; m += 8) {
          const float4 lo = *reinterpret_cast<const float4*>(tile_s + m * kSkBM + cg * 8);
          const float4 hi = *reinterpret_cast<const float4*>(tile_s + m * kSkBM + cg * 8 + 4);
          const float f[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
          for (int r = 0; r < p.os.world; ++r) {
            uint2* dst = p.os.slots_peer[r] + mine + (size_t)m * kSkBM;
            // two self-validating words per 16-byte store: halves the number of NVLink packets, and a store that the
            // fabric split in two would still deliver two consistent words
#pragma unroll
            for (int e = 0; e < 8; e += 2)
              st_relaxed_sys_v4(dst + e, __float_as_uint(f[e]), os_epoch, __float_as_uint(f[e + 1]), os_epoch);
          }
        }
      }
      SK_STAMP(5, tile == 0 && et == 0);
      if (ok && col < p.N) {
        float bias8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (p.bias) {
          const uint4 braw = *reinterpret_cast<const uint4*>(p.bias + col);
          const float2 b0 = unpack_bf16x2(braw.x), b1 = unpack_bf16x2(braw.y), b2 = unpack_bf16x2(braw.z),
                       b3 = unpack_bf16x2(braw.w);
          bias8[0] = b0.x; bias8[1] = b0.y; bias8[2] = b1.x; bias8[3] = b1.y;
          bias8[4] = b2.x; bias8[5] = b2.y; bias8[6] = b3.x; bias8[7] = b3.y;
        }
        for (int m = et >> 4; m < p.M && ok; m += 8) {
          float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int r = 0; r < p.os.world && ok; ++r) {    // fixed rank order: every rank computes the same bits
            const uint2* src = p.os.slots_local + half_off + (size_t)r * rank_stride + in_tile + (size_t)m * kSkBM;
            uint2 w[8];
            uint64_t t0 = 0;
            uint32_t spins = 0;
            while (true) {
              bool all = true;
#pragma unroll
              for (int e = 0; e < 8; e += 2) {
                const uint4 q4 = ld_relaxed_sys_v4(src + e);
                w[e] = make_uint2(q4.x, q4.y);
                w[e + 1] = make_uint2(q4.z, q4.w);
                all = all && (q4.y == os_epoch) && (q4.w == os_epoch);
              }
              if (all) break;
              if ((++spins & 0x3f) == 0) {
                if (*abort_flag) { ok = false; break; }
                const uint64_t now = global_timer_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > kWaitLimitNs) {
                  *abort_flag = 1;
                  report_error(kWaitFlagTimeout);
                  ok = false;
                  break;
                }
              }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += __uint_as_float(w[e].x);
          }
          if (!ok) break;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += bias8[e];
          if (p.residual) {
            const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + (long long)m * p.ldr + col);
            const float2 r0 = unpack_bf16x2(rr.x), r1 = unpack_bf16x2(rr.y), r2 = unpack_bf16x2(rr.z), r3 = unpack_bf16x2(rr.w);
            acc[0] += r0.x; acc[1] += r0.y; acc[2] += r1.x; acc[3] += r1.y;
            acc[4] += r2.x; acc[5] += r2.y; acc[6] += r3.x; acc[7] += r3.y;
          }
          uint4 o;
          o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
          o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
          *reinterpret_cast<uint4*>(p.C + (long long)m * p.ldc + col) = o;
        }
      }
      SK_STAMP(7, tile == 0 && et == 0);
    } else if (have_tile) {
      // Local tile -> symmetric partial buffer [tile][m][128]; flag the owner; the owner reduces and broadcasts.
      __nv_bfloat16* ptile = p.ar.partial + (size_t)tile * (MP * kSkBM);
#pragma unroll
      for (int m = 0; m < MP; ++m) ptile[m * kSkBM + n_local] = __float2bfloat16(v[m]);
      __threadfence_system();
      ok = epi_sync();
      const int owner = tile % p.ar.world;
      if (ok && et == 0) st_release_sys(p.ar.flags_peer[owner] + (size_t)tile * kMaxRanks + p.ar.rank, ar_epoch);
      if (ok && owner == p.ar.rank) {
        bool got = true;
        if (lane < p.ar.world)
          got = wait_flag_ge(p.ar.flags_peer[p.ar.rank] + (size_t)tile * kMaxRanks + lane, ar_epoch);
        if (!__all_sync(0xffffffffu, got)) {
          *abort_flag = 1;
        } else {
          // 16 lanes cover one output row's 128 columns (8 each); the 128 threads take 8 rows per pass.
          const int cg = et & 15;
          const int col = n0 + cg * 8;
          if (col < p.N) {
            float bias8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (p.bias) {
              const uint4 braw = *reinterpret_cast<const uint4*>(p.bias + col);
              const float2 b0 = unpack_bf16x2(braw.x), b1 = unpack_bf16x2(braw.y), b2 = unpack_bf16x2(braw.z),
                           b3 = unpack_bf16x2(braw.w);
              bias8[0] = b0.x; bias8[1] = b0.y; bias8[2] = b1.x; bias8[3] = b1.y;
              bias8[4] = b2.x; bias8[5] = b2.y; bias8[6] = b3.x; bias8[7] = b3.y;
            }
            for (int m = et >> 4; m < p.M; m += 8) {
              const long long off = (long long)tile * (MP * kSkBM) + (long long)m * kSkBM + cg * 8;
              float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
              auto add8 = [&](const uint4& u) {
                const float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z),
                             a3 = unpack_bf16x2(u.w);
                acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y;
                acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
              };
              if (p.ar.use_nvls) {
                add8(multimem_ld_reduce_bf16x8(p.ar.mc_partial + off));
              } else {
                for (int r = 0; r < p.ar.world; ++r) add8(ld_cg_v4(p.ar.peer_partial[r] + off));
              }
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[e] += bias8[e];
              if (p.residual) add8(*reinterpret_cast<const uint4*>(p.residual + (long long)m * p.ldr + col));
              uint4 o;
              o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
              o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
              const long long o_off = (long long)m * p.ldc + col;
              if (p.ar.use_nvls) {
                multimem_st_bf16x8(p.ar.mc_out + o_off, o);
              } else {
                for (int r = 0; r < p.ar.world; ++r) st_cg_v4(p.ar.out_peer[r] + o_off, o);
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
  if (p.os.world > 0 && threadIdx.x == 0) {
    // Launch counter of the one-shot protocol: advanced by the last CTA to leave (no cross-rank handshake).
    __threadfence();
    if (atomicAdd(p.os.exit_counter, 1u) == gridDim.x - 1) {
      *p.os.exit_counter = 0;
      *p.os.epoch = os_epoch;
    }
  }
  if (p.ar.world > 0 && threadIdx.x == 0) {
    // This rank's output is final once every rank has finished the tiles it owns.
    __threadfence_system();
    if (atomicAdd(p.ar.exit_counter, 1u) == gridDim.x - 1) {
      *p.ar.exit_counter = 0;
      __threadfence_system();
      const size_t done0 = (size_t)p.ar.max_tiles * kMaxRanks;
      for (int r = 0; r < p.ar.world; ++r) st_release_sys(p.ar.flags_peer[r] + done0 + p.ar.rank, ar_epoch);
      for (int r = 0; r < p.ar.world; ++r)
        if (!wait_flag_ge(p.ar.flags_peer[p.ar.rank] + done0 + r, ar_epoch)) break;
      *p.ar.epoch = ar_epoch;
    }
  }
}

template <int MP>
static int launch_skinny(const CUtensorMap& tmW, const CUtensorMap& tmX, const SkinnyParams& p, int units,
                         cudaStream_t stream) {
  using L = SkinnySmem<MP>;
  auto kern = gemm_skinny_kernel<MP>;
  static bool configured = false;
  if (!configured) {
    DPTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    configured = true;
  }
  return counted(1, (int)launch_k(kern, dim3(units), dim3(kSkThreads), L::kTotal, stream, tmW, tmX, p));
}

}  // namespace dptb

using namespace dptb;

// Turns programmatic dependent launch on or off for the kernels of the decode step (this kernel, RMSNorm, rotary +
// cache append, decode attention, SwiGLU).  The caller keeps it on only around a chain in which the kernel before an
// all-reduce GEMM is never another all-reduce GEMM (this kernel reads its protocol counters before its wait).
extern "C" void dptb_gemm_skinny_set_pdl(int on) { dptb::pdl_flag() = on ? 1 : 0; }

// Peer-memory description of the one-shot all-reduce (see SkinnyOneShot); every rank's slot buffer holds
// 2 * kMaxRanks * max_tiles * 64 * 128 eight-byte words, zero-initialised.
struct DptbTpOneShotArgs {
  int world, rank, max_tiles, reserved;
  void* slots_peer[kDptbMaxRanks];
  void* epoch;
  void* exit_counter;
};

// Timeline stamps (see DPTB_SKINNY_PROFILE); -5 when not compiled in.
extern "C" int dptb_gemm_skinny_profile_read(unsigned long long* out) {
#ifdef DPTB_SKINNY_PROFILE
  return (int)cudaMemcpyFromSymbol(out, g_skinny_prof, sizeof(unsigned long long) * 8);
#else
  (void)out;
  return kErrUnsupported;
#endif
}

// out[M, N] = x[M, K] @ W[N, K]^T (+ bias) (+ residual), M <= 64, bf16 everywhere; with `ar` the sum over the ranks of a
// tensor-parallel group lands in every rank's output (C of the argument block is then ignored).  Returns
// kErrUnsupported for anything else, so callers can fall back to dptb_gemm / dptb_gemm_allreduce.
static int skinny_impl(const DptbGemmArgs* a, const DptbTpArArgs* ar, const DptbTpOneShotArgs* os, void* stream_v);
extern "C" int dptb_gemm_skinny(const DptbGemmArgs* a, const DptbTpArArgs* ar, void* stream_v) {
  return skinny_impl(a, ar, nullptr, stream_v);
}
// Same product with the one-shot all-reduce: the sum over the ranks (+ bias, + residual) is written to C of the
// argument block, which is this rank's own output buffer; every rank computes identical bits.
extern "C" int dptb_gemm_skinny_oneshot(const DptbGemmArgs* a, const DptbTpOneShotArgs* os, void* stream_v) {
  if (!os) return kErrBadShape;
  return skinny_impl(a, nullptr, os, stream_v);
}
static int skinny_impl(const DptbGemmArgs* a, const DptbTpArArgs* ar, const DptbTpOneShotArgs* os, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (a->M <= 0 || a->N <= 0) return 0;
  if (a->M > 64 || a->K <= 0 || a->trans_a || !a->trans_b || a->a_f32 || a->b_f32 || a->out_f32 || a->accumulate ||
      a->act || a->aux_out || a->aux_in || a->alpha != 1.0f || (a->bias && a->bias_f32))
    return kErrUnsupported;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!al16(a->A) || !al16(a->B) || (a->lda % 8) || (a->ldb % 8)) return kErrUnsupported;
  if (ar) {
    if (ar->mode != 0 || ar->world < 1 || ar->world > kMaxRanks || ar->rank < 0 || ar->rank >= ar->world)
      return kErrUnsupported;
    if ((a->N % 8) || (a->ldc % 8) || (a->bias && !al16(a->bias)) ||
        (a->residual && (!al16(a->residual) || a->ldr % 8)))
      return kErrUnsupported;
  }
  if (os) {
    if (os->world < 1 || os->world > kMaxRanks || os->rank < 0 || os->rank >= os->world) return kErrUnsupported;
    if (!al16(a->C) || (a->N % 8) || (a->ldc % 8) || (a->bias && !al16(a->bias)) ||
        (a->residual && (!al16(a->residual) || a->ldr % 8)))
      return kErrUnsupported;
  }
  const int mp = a->M <= 32 ? 32 : 64;
  const int tiles = (a->N + kSkBM - 1) / kSkBM;
  const int num_kb = (a->K + kSkBK - 1) / kSkBK;
  // Split K so that the work units fill the SMs once, with at least 4 k-blocks each.
  int splits = a->splits >= 1 ? a->splits : 1;
  if (a->splits < 1) {
    static const int min_kb = [] {
      const char* e = getenv("DPTB_SKINNY_MIN_KB");
      const int v = e ? atoi(e) : 0;
      return v > 0 ? v : 4;
    }();
    const int by_sm = sm_count() / tiles;
    const int by_k = num_kb / min_kb;
    splits = by_sm < by_k ? by_sm : by_k;
    if (splits < 1) splits = 1;
  }
  if (splits > 1) {
    const bool have_ws = a->ws && a->counters && tiles <= a->num_counters &&
                         (long long)tiles * splits * mp * kSkBM * 4 <= a->ws_bytes;
    if (!have_ws) splits = 1;
  }
  int kb_per_split = (num_kb + splits - 1) / splits;
  splits = (num_kb + kb_per_split - 1) / kb_per_split;   // every split non-empty
  SkinnyParams p;
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.C = static_cast<__nv_bfloat16*>(a->C); p.ldc = a->ldc;
  p.bias = static_cast<const __nv_bfloat16*>(a->bias);
  p.residual = static_cast<const __nv_bfloat16*>(a->residual); p.ldr = a->ldr;
  p.num_kb = num_kb; p.splits = splits; p.kb_per_split = kb_per_split;
  p.vec_out = (al16(a->C) && a->ldc % 8 == 0 && a->N % 8 == 0 &&
               (!a->residual || (al16(a->residual) && a->ldr % 8 == 0))) ? 1 : 0;
  p.ws = static_cast<float*>(a->ws);
  p.counters = a->counters;
  p.ar.world = 0;
  p.os.world = 0;
  if (os) {
    if (tiles > os->max_tiles) return kErrTooLarge;
    p.os.world = os->world; p.os.rank = os->rank;
    p.os.slots_local = static_cast<uint2*>(os->slots_peer[os->rank]);
    for (int r = 0; r < kMaxRanks; ++r) p.os.slots_peer[r] = static_cast<uint2*>(os->slots_peer[r]);
    p.os.max_tiles = os->max_tiles;
    p.os.epoch = static_cast<uint32_t*>(os->epoch);
    p.os.exit_counter = static_cast<unsigned int*>(os->exit_counter);
  }
  if (ar) {
    if (tiles > ar->max_tiles || (long long)tiles * mp * kSkBM > ar->partial_elems) return kErrTooLarge;
    p.ar.world = ar->world; p.ar.rank = ar->rank;
    p.ar.use_nvls = (ar->use_nvls && ar->mc_partial && ar->mc_out) ? 1 : 0;
    p.ar.partial = static_cast<__nv_bfloat16*>(ar->partial);
    p.ar.mc_partial = static_cast<const __nv_bfloat16*>(ar->mc_partial);
    p.ar.mc_out = static_cast<__nv_bfloat16*>(ar->mc_out);
    for (int r = 0; r < kMaxRanks; ++r) {
      p.ar.peer_partial[r] = static_cast<const __nv_bfloat16*>(ar->peer_partial[r]);
      p.ar.out_peer[r] = static_cast<__nv_bfloat16*>(ar->out_peer[r]);
      p.ar.flags_peer[r] = static_cast<uint32_t*>(ar->flags_peer[r]);
    }
    p.ar.max_tiles = ar->max_tiles;
    p.ar.epoch = static_cast<uint32_t*>(ar->epoch);
    p.ar.exit_counter = static_cast<unsigned int*>(ar->exit_counter);
  }
  CUtensorMap tmW, tmX;
  int rc = encode_tmap_2d_bf16(&tmW, a->B, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->ldb * 2, 64, kSkBM);
  if (rc) return rc;
  rc = encode_tmap_2d_bf16(&tmX, a->A, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->lda * 2, 64, (uint32_t)mp);
  if (rc) return rc;
  const int units = tiles * splits;
  return mp == 32 ? launch_skinny<32>(tmW, tmX, p, units, stream) : launch_skinny<64>(tmW, tmX, p, units, stream);
}
