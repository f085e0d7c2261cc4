// bf16 GEMM on 5th-generation tensor cores (tcgen05 + TMEM) with fused epilogues, plus a plain
// SIMT kernel for shapes / dtypes the tensor-core path cannot take.
//
//   C[M,N] = epilogue( op(A)[M,K] * op(B)[K,N] )
//
// It replaces the reference's single 32x32 shared-memory-tiled fp32 matmul and the transpose /
// row-broadcast-add / activation kernels around it (reference: lib/native/src/kernels/matmul.cuh:27-63,
// lib/native/src/kernels/transpose.cuh:12-29, lib/native/src/kernels/elementwise.cuh:64-73).
//
// Structure of the tensor-core kernel (one persistent CTA per SM, 320 threads):
//   warp 0      TMA producer: one elected lane streams 128xBK / BNxBK tiles into a STAGES-deep ring.
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma (M=128, N=BN, K=16) into one of two
//               TMEM accumulators; tcgen05.commit releases smem stages and publishes accumulators.
//   warps 2-9   epilogue (two warps per TMEM lane quarter, alternating 64-column blocks): tcgen05.ld of the
//               finished accumulator (one row per thread), bias / activation / residual / accumulate in
//               registers, bf16 or fp32 stores, while the issuer already works on the next tile in the
//               other accumulator.
#include <cuda_bf16.h>

#include "common/gemm_args.h"
#include "common/host.h"
#include "common/peer.cuh"
#include "common/ptx.cuh"

namespace dptb {

// Opt-in role timers (compile with -DDPTB_GEMM_PROFILE): per CTA, SM clock cycles each warp role spent waiting.
//   [0] producer waiting for a free stage   [1] producer total
//   [2] issuer waiting for a loaded stage   [3] issuer waiting for a free accumulator   [4] issuer total
//   [5] epilogue warp 0 waiting for a finished accumulator   [6] epilogue warp 0 total   [7] work units
//   [8] epilogue warp 0: accumulator loads (TMEM -> registers)   [9] epilogue warp 0: math + stores   [10] blocks
#ifdef DPTB_GEMM_PROFILE
constexpr int kProfSlots = 12;
__device__ unsigned long long g_gemm_prof[256][kProfSlots];
#define DPTB_PROF_DECL(name) long long name = 0
#define DPTB_PROF_BEGIN(t) const long long t = clock64()
#define DPTB_PROF_END(t, acc) acc += clock64() - t
#define DPTB_PROF_STORE(slot, v) g_gemm_prof[blockIdx.x & 255][slot] += (unsigned long long)(v)
#else
#define DPTB_PROF_DECL(name)
#define DPTB_PROF_BEGIN(t)
#define DPTB_PROF_END(t, acc)
#define DPTB_PROF_STORE(slot, v)
#endif

// Registry of the per-translation-unit status blocks (filled by static initialisers at load time).
static int (*g_status_blocks[64])(int*, int);
static int g_num_status_blocks = 0;
void register_status_block(int (*access)(int*, int)) {
  if (g_num_status_blocks < 64) g_status_blocks[g_num_status_blocks++] = access;
}

// Tensor-parallel all-reduce epilogue (row-parallel Linear: every rank holds a K-slice of the weight and produces a
// partial [M, N]; the sum over ranks, plus bias / residual, must reach every rank).  world == 0 switches it off.
//
// All ranks launch the same grid over the same tiles.  A CTA stores the bf16 partial of tile t into this rank's
// `partial` buffer (layout [tile][64-column chunk][128 rows][64]), then raises ready[t][rank] in the flag array of the
// tile's owner, rank t % world.  On the owner, the epilogue warps of the CTA that computed tile t wait (bounded) for
// all `world` flags, sum the partials in rank order -- one multimem.ld_reduce per 16 bytes through the NVSwitch when a
// multicast mapping exists, else one peer load per rank -- add bias and residual, and write the result into every
// rank's output (multimem.st, else one peer store per rank).  The MMA warp meanwhile works on the next tile in the
// other TMEM accumulator, so NVLink traffic of tile t overlaps the tensor-core work of tile t + gridDim.x.  At the end
// the last CTA of each rank raises done[rank] on every peer and waits for all done flags: when a rank's kernel
// completes, its whole output is final.  Epochs count launches, so no flag is ever reset and CUDA graphs can replay.
struct TpAr {
  int world, rank;
  int use_nvls;
  __nv_bfloat16* partial;                   // local
  const __nv_bfloat16* peer_partial[kMaxRanks];
  const __nv_bfloat16* mc_partial;          // multicast view of the partial buffers (or null)
  __nv_bfloat16* out_peer[kMaxRanks];       // every rank's output [M, ldc]
  __nv_bfloat16* mc_out;                    // multicast view of the outputs (or null)
  uint32_t* flags_peer[kMaxRanks];          // every rank's flags: ready[max_tiles][kMaxRanks] then done[kMaxRanks]
  int max_tiles;
  uint32_t* epoch;                          // local launch counter
  unsigned int* exit_counter;               // local, zero between launches
  // mode 1 = reduce-scatter by rows (sequence-parallel output): rank r keeps rows [r * M / world, (r + 1) * M / world)
  // of the sum in ITS output only (row 0 of that buffer = first row of the shard; bias / residual are indexed the same
  // way).  The owner of a tile is then the rank that keeps its rows, and the row tiles are visited round-robin over
  // the owners so that every rank's reductions are spread over the whole kernel.
  int mode;
  int rows_per_rank;
};

// All-gather prologue (column-parallel Linear on a row-sharded input): the A operand of row tile i is read by TMA from
// the symmetric buffer of the rank that owns those rows (a plain, non-multicast tile load over NVLink; its own rows come
// from local memory), after that rank's "shard ready" flag has reached the expected launch number.  world == 0: off.
struct TpAg {
  int world, rank;
  int tiles_per_rank;                       // 128-row tiles per shard
  const uint32_t* ready;                    // local flags [kMaxRanks], written by the peers' signal kernels
  const uint32_t* epoch;                    // local word: the value ready[r] must have reached
};
struct TmapSet {
  CUtensorMap m[kMaxRanks];
};

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const void* bias;       // [N], fp32 or bf16
  int bias_f32;
  const __nv_bfloat16* residual;  // [M, ldr]
  long long ldr;
  __nv_bfloat16* aux_out;         // pre-activation copy [M, ld_aux_out]
  long long ld_aux_out;
  const __nv_bfloat16* aux_in;    // pre-activation input for the derivative modes [M, ld_aux_in]
  long long ld_aux_in;
  int act;         // 0 none 1 relu 2 gelu_tanh 3 quick_gelu 4 silu | 11..14: multiply by act'(aux_in)
  int out_f32;     // C is float
  int accumulate;  // C += result
  float alpha;
  int vec_ok;      // all pointers 16-byte aligned and leading dimensions multiples of 8 elements
  int row_epi;     // row-per-thread register epilogue for bf16 C: 0 off (staged), 1 = 16-byte, 2 = 32-byte accesses
  int tiles_m, tiles_n, num_kb;
  // Split-K: each tile's K range is cut into `splits` work units of kb_per_split k-blocks; partial accumulators go
  // through `ws` (fp32, [tile][split][BN][128]) and the last unit of a tile to finish (per-tile counter) folds them in
  // split order, so the result does not depend on arrival order.
  int splits, kb_per_split;
  float* ws;
  int* counters;
  TpAr ar;
  TpAg ag;
};

// Row-tile index of work unit `tile` after the tensor-parallel re-orderings (identity otherwise).
//   reduce-scatter: consecutive row tiles go to consecutive owners;
//   all-gather:     every rank starts with its own shard and then walks the ring, so that at any moment the ranks pull
//                   from different peers.
__device__ __forceinline__ int tile_row_index(const GemmParams& p, int tile) {
  int mi = tile % p.tiles_m;
  if (p.ar.world > 0 && p.ar.mode == 1) {
    const int tpr = p.tiles_m / p.ar.world;
    mi = (mi % p.ar.world) * tpr + mi / p.ar.world;
  } else if (p.ag.world > 0) {
    const int tpr = p.ag.tiles_per_rank;
    mi = ((mi / tpr + p.ag.rank) % p.ag.world) * tpr + mi % tpr;
  }
  return mi;
}

// ----------------------------------------------------------------------------- epilogue math
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sigmoid_fast(float x) { return 1.0f / (1.0f + __expf(-x)); }

__device__ __forceinline__ float act_fwd(int act, float x) {
  switch (act) {
    case 1: return fmaxf(x, 0.0f);
    case 2:
    case 5: {
      float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + tanh_fast(u));
    }
    case 3: return x * sigmoid_fast(1.702f * x);
    case 4: return x * sigmoid_fast(x);
    default: return x;
  }
}
__device__ __forceinline__ float act_bwd(int act, float x) {
  switch (act) {
    case 11: return x > 0.0f ? 1.0f : 0.0f;
    case 12: {
      float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      float t = tanh_fast(u);
      return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x * x);
    }
    case 13: {
      float s = sigmoid_fast(1.702f * x);
      return s + 1.702f * x * s * (1.0f - s);
    }
    case 14: {
      float s = sigmoid_fast(x);
      return s * (1.0f + x * (1.0f - s));
    }
    case 15: return x;   // the saved tensor already is the derivative (see act code 5)
    default: return 1.0f;
  }
}
// What the auxiliary output receives: the pre-activation value, or (act code 5, the training MLP) the GELU derivative
// at that value, so that the backward GEMM's epilogue is one multiply per element instead of a second tanh.
__device__ __forceinline__ float aux_value(int act, float x) { return act == 5 ? act_bwd(12, x) : x; }

// One output element, used by the tail path of the tensor-core kernel and by the SIMT kernel.
__device__ __forceinline__ void epilogue_scalar(const GemmParams& p, long long row, long long col, float v) {
  v *= p.alpha;
  if (p.bias) v += p.bias_f32 ? static_cast<const float*>(p.bias)[col] : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col]);
  if (p.aux_out) p.aux_out[row * p.ld_aux_out + col] = __float2bfloat16(aux_value(p.act, v));
  if (p.act >= 1 && p.act <= 5) v = act_fwd(p.act, v);
  if (p.act >= 11) v *= act_bwd(p.act, __bfloat162float(p.aux_in[row * p.ld_aux_in + col]));
  if (p.residual) v += __bfloat162float(p.residual[row * p.ldr + col]);
  if (p.out_f32) {
    float* c = static_cast<float*>(p.C) + row * p.ldc + col;
    *c = p.accumulate ? *c + v : v;
  } else {
    __nv_bfloat16* c = static_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col;
    *c = __float2bfloat16(p.accumulate ? __bfloat162float(*c) + v : v);
  }
}

// Activation (or activation-derivative multiply) on 8 values, dispatched once per group so the loops stay branch-free.
__device__ __forceinline__ void apply_act8(int act, float (&v)[8]) {
  switch (act) {
    case 1:
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = fmaxf(v[i], 0.0f);
      break;
    case 2:
    case 5:
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float x = v[i];
        v[i] = 0.5f * x * (1.0f + tanh_fast(0.7978845608028654f * fmaf(0.044715f * x * x, x, x)));
      }
      break;
    case 3:
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __fdividef(v[i], 1.0f + __expf(-1.702f * v[i]));
      break;
    case 4:
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __fdividef(v[i], 1.0f + __expf(-v[i]));
      break;
    default: break;
  }
}
__device__ __forceinline__ void apply_act_bwd8(int act, float (&v)[8], const float (&x)[8]) {
  switch (act) {
    case 11:
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = x[i] > 0.0f ? v[i] : 0.0f;
      break;
    case 12:
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xx = x[i] * x[i];
        const float t = tanh_fast(0.7978845608028654f * fmaf(0.044715f * xx, x[i], x[i]));
        const float d = 0.5f * (1.0f + t) + 0.5f * x[i] * (1.0f - t * t) * (0.7978845608028654f + 0.1070322243f * xx);
        v[i] *= d;
      }
      break;
    case 13:
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float sg = __fdividef(1.0f, 1.0f + __expf(-1.702f * x[i]));
        v[i] *= sg + 1.702f * x[i] * sg * (1.0f - sg);
      }
      break;
    case 14:
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float sg = __fdividef(1.0f, 1.0f + __expf(-x[i]));
        v[i] *= sg * (1.0f + x[i] * (1.0f - sg));
      }
      break;
    case 15:
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] *= x[i];
      break;
    default: break;
  }
}
__device__ __forceinline__ void aux_value8(int act, const float (&v)[8], float (&o)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = aux_value(act, v[i]);
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// Second phase of the staged epilogue.  `stage` holds a 32-row x 64-column bf16 block of alpha-scaled accumulators (rows
// 128 bytes, 16-byte chunks XOR-swizzled by row).  Lanes are re-mapped so that 8 lanes cover one row's 128 bytes:
// every global access of the warp is 4 full 128-byte row segments.  bias -> aux_out -> act -> act' -> residual -> (+C) -> C.
__device__ __forceinline__ void epilogue_phase2(const GemmParams& p, const uint8_t* stage, long long row0, long long col0,
                                                int lane) {
  const int rg = lane >> 3, cg = lane & 7;
  const long long col = col0 + cg * 8;
  const bool full = p.vec_ok && (col0 + 64 <= p.N);
  float bias8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (p.bias) {
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (col + e < p.N)
        bias8[e] = p.bias_f32 ? __ldg(static_cast<const float*>(p.bias) + col + e)
                              : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col + e]);
  }
  __nv_bfloat16* C = static_cast<__nv_bfloat16*>(p.C);
#pragma unroll 2
  for (int it = 0; it < 8; ++it) {
    const int rl = it * 4 + rg;
    const long long row = row0 + rl;
    if (row >= p.M) continue;
    const uint4 raw = *reinterpret_cast<const uint4*>(stage + rl * 128 + ((cg ^ (rl & 7)) << 4));
    float v[8];
    unpack8(raw, v);
    if (p.bias) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += bias8[e];
    }
    if (full) {
      if (p.aux_out) {
        float av[8];
        aux_value8(p.act, v, av);
        *reinterpret_cast<uint4*>(p.aux_out + row * p.ld_aux_out + col) = pack8(av);
      }
      if (p.act >= 1 && p.act <= 5) apply_act8(p.act, v);
      if (p.act >= 11) {
        float x[8];
        unpack8(*reinterpret_cast<const uint4*>(p.aux_in + row * p.ld_aux_in + col), x);
        apply_act_bwd8(p.act, v, x);
      }
      if (p.residual) {
        float r[8];
        unpack8(*reinterpret_cast<const uint4*>(p.residual + row * p.ldr + col), r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += r[e];
      }
      if (p.accumulate) {
        float o[8];
        unpack8(*reinterpret_cast<const uint4*>(C + row * p.ldc + col), o);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += o[e];
      }
      *reinterpret_cast<uint4*>(C + row * p.ldc + col) = pack8(v);
    } else {
      float x[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (col + e < p.N) {
          if (p.aux_out) p.aux_out[row * p.ld_aux_out + col + e] = __float2bfloat16(aux_value(p.act, v[e]));
          if (p.act >= 11) x[e] = __bfloat162float(p.aux_in[row * p.ld_aux_in + col + e]);
        }
      if (p.act >= 1 && p.act <= 5) apply_act8(p.act, v);
      if (p.act >= 11) apply_act_bwd8(p.act, v, x);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (col + e < p.N) {
          float o = v[e];
          if (p.residual) o += __bfloat162float(p.residual[row * p.ldr + col + e]);
          if (p.accumulate) o += __bfloat162float(C[row * p.ldc + col + e]);
          C[row * p.ldc + col + e] = __float2bfloat16(o);
        }
    }
  }
}

// fp32-output epilogue for 32 consecutive columns of one row straight from registers (row-per-thread mapping).
__device__ __forceinline__ void epilogue_direct_f32(const GemmParams& p, long long row, long long col,
                                                    const uint32_t (&r)[32]) {
  const bool full = p.vec_ok && (col + 32 <= p.N);
  float* C = static_cast<float*>(p.C) + row * p.ldc + col;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float v[8], x[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      v[e] = __uint_as_float(r[g * 8 + e]) * p.alpha;
      const long long c = col + g * 8 + e;
      if (c < p.N) {
        if (p.bias) v[e] += p.bias_f32 ? __ldg(static_cast<const float*>(p.bias) + c)
                                       : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[c]);
        if (p.aux_out) p.aux_out[row * p.ld_aux_out + c] = __float2bfloat16(aux_value(p.act, v[e]));
        if (p.act >= 11) x[e] = __bfloat162float(p.aux_in[row * p.ld_aux_in + c]);
      }
    }
    if (p.act >= 1 && p.act <= 5) apply_act8(p.act, v);
    if (p.act >= 11) apply_act_bwd8(p.act, v, x);
    if (full) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float4 o = make_float4(v[h * 4], v[h * 4 + 1], v[h * 4 + 2], v[h * 4 + 3]);
        if (p.residual) {
          const __nv_bfloat16* rr = p.residual + row * p.ldr + col + g * 8 + h * 4;
          o.x += __bfloat162float(rr[0]); o.y += __bfloat162float(rr[1]);
          o.z += __bfloat162float(rr[2]); o.w += __bfloat162float(rr[3]);
        }
        float4* dst = reinterpret_cast<float4*>(C + g * 8 + h * 4);
        if (p.accumulate) {
          const float4 c4 = *dst;
          o.x += c4.x; o.y += c4.y; o.z += c4.z; o.w += c4.w;
        }
        *dst = o;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const long long c = col + g * 8 + e;
        if (c < p.N) {
          float o = v[e];
          if (p.residual) o += __bfloat162float(p.residual[row * p.ldr + c]);
          if (p.accumulate) o += C[g * 8 + e];
          C[g * 8 + e] = o;
        }
      }
    }
  }
}

// ----------------------------------------------------------------------------- row-per-thread epilogue
// One 32-row x 64-column block of a bf16 output.  Each thread owns one row (the TMEM mapping) and keeps its 64 values
// in registers through the whole epilogue: no shared-memory round trip, no warp synchronisation, and every stage
// (scale, bias, activation, residual, ...) is one fully unrolled pass over the 64 values behind a warp-uniform branch,
// so the loads, conversions and stores of a stage are independent and overlap.  A thread reads and writes its row in
// 32-byte pieces (whole sectors) when the buffers allow it, else in 16-byte pieces.  Measured with the role timers of
// this file, the staged variant (registers -> shared memory -> lanes re-mapped to whole 128-byte lines) spends about
// 3700 cycles per block on dependent shared-memory round trips; a variant that handed the staged block to a TMA tile
// store was slower still (it waits for the copy engine to drain the staging block).
struct EpiIn {
  uint4 v[8];
  int kind;   // 0 none, 1 aux_in, 2 residual, 3 C (accumulate)
};
__device__ __forceinline__ void ld_row64(const __nv_bfloat16* s, bool wide, uint4 (&v)[8]) {
  if (wide) {
#pragma unroll
    for (int g = 0; g < 4; ++g)
      asm volatile("ld.global.L1::no_allocate.v8.u32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                   : "=r"(v[2 * g].x), "=r"(v[2 * g].y), "=r"(v[2 * g].z), "=r"(v[2 * g].w), "=r"(v[2 * g + 1].x),
                     "=r"(v[2 * g + 1].y), "=r"(v[2 * g + 1].z), "=r"(v[2 * g + 1].w)
                   : "l"(s + g * 16));
  } else {
#pragma unroll
    for (int g = 0; g < 8; ++g) v[g] = ld_stream_v4(s + g * 8);
  }
}
__device__ __forceinline__ void st_row64(__nv_bfloat16* d, bool wide, const uint4 (&v)[8]) {
  if (wide) {
#pragma unroll
    for (int g = 0; g < 4; ++g)
      asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                   ::"l"(d + g * 16), "r"(v[2 * g].x), "r"(v[2 * g].y), "r"(v[2 * g].z), "r"(v[2 * g].w),
                   "r"(v[2 * g + 1].x), "r"(v[2 * g + 1].y), "r"(v[2 * g + 1].z), "r"(v[2 * g + 1].w)
                   : "memory");
  } else {
#pragma unroll
    for (int g = 0; g < 8; ++g) *reinterpret_cast<uint4*>(d + g * 8) = v[g];
  }
}
__device__ __forceinline__ void add_row64(float (&v)[64], const uint4 (&t)[8]) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    float f[8];
    unpack8(t[g], f);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[g * 8 + e] += f[e];
  }
}
// Tensor maps of the tile-store epilogue (32-row x 64-column bf16 boxes, 128-byte swizzle): the output, the optional
// pre-activation copy, and the one optional per-element input (activation input, residual, or C itself when
// accumulating).  Unused maps are copies of the output's.
struct EpiMaps {
  CUtensorMap c, aux, in;
};
// One thread's 128-byte row of a staged 32 x 64 block, 16-byte chunks XOR-swizzled by row as the tile copies expect.
__device__ __forceinline__ void st_smem_row64(uint8_t* buf, int lane, const uint4 (&v)[8]) {
  uint8_t* row = buf + lane * 128;
#pragma unroll
  for (int g = 0; g < 8; ++g) *reinterpret_cast<uint4*>(row + ((g ^ (lane & 7)) << 4)) = v[g];
}
__device__ __forceinline__ void ld_smem_row64(const uint8_t* buf, int lane, uint4 (&v)[8]) {
  const uint8_t* row = buf + lane * 128;
#pragma unroll
  for (int g = 0; g < 8; ++g) v[g] = *reinterpret_cast<const uint4*>(row + ((g ^ (lane & 7)) << 4));
}
// Wait until at most one of this thread's tile stores is still reading its shared-memory source.
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

// Requests the first per-element input of the block (and the bias slice) before the accumulator load is waited for.
__device__ __forceinline__ void epi_prefetch(const GemmParams& p, uint32_t* bias_s, long long row, long long col0,
                                             int lane, EpiIn& in) {
  const __nv_bfloat16* src = nullptr;
  long long ld = 0;
  in.kind = 0;
  if (p.act >= 11) { src = p.aux_in; ld = p.ld_aux_in; in.kind = 1; }
  else if (p.residual) { src = p.residual; ld = p.ldr; in.kind = 2; }
  else if (p.accumulate) { src = static_cast<const __nv_bfloat16*>(p.C); ld = p.ldc; in.kind = 3; }
  if (in.kind != 0 && row < p.M) {
    ld_row64(src + row * ld + col0, p.row_epi == 2, in.v);
  } else {
#pragma unroll
    for (int g = 0; g < 8; ++g) in.v[g] = make_uint4(0, 0, 0, 0);
  }
  if (p.bias) bias_s[lane] = __ldg(reinterpret_cast<const uint32_t*>(static_cast<const __nv_bfloat16*>(p.bias) + col0) + lane);
}
__device__ __forceinline__ void epi_finish_row(const GemmParams& p, const uint32_t* bias_s, long long row0,
                                               long long col0, int lane, const uint32_t (&r0)[32],
                                               const uint32_t (&r1)[32], const EpiIn& in) {
  const long long row = row0 + lane;
  const bool live = row < p.M;
  const bool wide = p.row_epi == 2;
  float v[64];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    v[i] = __uint_as_float(r0[i]);
    v[32 + i] = __uint_as_float(r1[i]);
  }
  if (p.alpha != 1.0f) {
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] *= p.alpha;
  }
  if (p.bias) {
    __syncwarp();   // the bias slice written by epi_prefetch is visible
    uint4 b[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) b[g] = *reinterpret_cast<const uint4*>(bias_s + g * 4);
    add_row64(v, b);
    __syncwarp();   // all lanes have read it before the next block overwrites it
  }
  if (p.aux_out) {
    uint4 o[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float av[8];
      aux_value8(p.act, reinterpret_cast<const float(&)[8]>(v[g * 8]), av);
      o[g] = pack8(av);
    }
    if (live) st_row64(p.aux_out + row * p.ld_aux_out + col0, wide, o);
  }
  if (p.act == 2 || p.act == 5) {
    // GELU (tanh form), the one activation on the training hot path, outside the per-group dispatch: five
    // multiply-adds and one tanh.approx per element, all 64 elements independent.
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      const float x = v[i];
      const float u = x * fmaf(x * x, 0.0356774081f, 0.7978845608f);   // 0.79788456 (x + 0.044715 x^3)
      const float hx = 0.5f * x;
      v[i] = fmaf(hx, tanh_fast(u), hx);
    }
  } else if (p.act >= 1 && p.act <= 5) {
#pragma unroll
    for (int g = 0; g < 8; ++g) apply_act8(p.act, reinterpret_cast<float(&)[8]>(v[g * 8]));
  }
  if (p.act == 12) {
    // GELU (tanh form) derivative, outside the per-group dispatch like the forward:
    //   d = 0.5 (1 + t) + 0.5 x (1 - t^2) (0.79788456 + 0.10703222 x^2),  t = tanh(0.79788456 (x + 0.044715 x^3))
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float x[8];
      unpack8(in.v[g], x);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float xx = x[e] * x[e];
        const float t = tanh_fast(x[e] * fmaf(xx, 0.0356774081f, 0.7978845608f));
        const float s = x[e] * fmaf(xx, 0.1070322243f, 0.7978845608f);
        v[g * 8 + e] *= 0.5f * (1.0f + t + s * fmaf(-t, t, 1.0f));
      }
    }
  } else if (p.act >= 11) {
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float x[8];
      unpack8(in.v[g], x);
      apply_act_bwd8(p.act, reinterpret_cast<float(&)[8]>(v[g * 8]), x);
    }
  }
  if (p.residual) {
    if (in.kind == 2) {
      add_row64(v, in.v);
    } else {
      uint4 t[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) t[g] = make_uint4(0, 0, 0, 0);
      if (live) ld_row64(p.residual + row * p.ldr + col0, wide, t);
      add_row64(v, t);
    }
  }
  if (p.accumulate) {
    if (in.kind == 3) {
      add_row64(v, in.v);
    } else {
      uint4 t[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) t[g] = make_uint4(0, 0, 0, 0);
      if (live) ld_row64(static_cast<const __nv_bfloat16*>(p.C) + row * p.ldc + col0, wide, t);
      add_row64(v, t);
    }
  }
  uint4 o[8];
#pragma unroll
  for (int g = 0; g < 8; ++g) o[g] = pack8(reinterpret_cast<const float(&)[8]>(v[g * 8]));
  if (live) st_row64(static_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0, wide, o);
}

// Tile-store epilogue, one half (32 columns) of a thread's row at a time so that the values, the per-element input and
// the packed output of a half fit in registers together.  `r` holds the accumulators of columns [32 h, 32 h + 32) of the
// 64-column block; the input (if any) is read from, and the output written to, chunks 4 h .. 4 h + 3 of the thread's
// row in the swizzled staging blocks.  bias -> (copy to buf_aux) -> activation -> activation' -> + input -> buf_c.
__device__ __forceinline__ void epi_half_tma(const GemmParams& p, const uint32_t* bias_s, int h, int lane, int in_kind,
                                             const uint32_t (&r)[32], uint8_t* buf_aux, uint8_t* buf_c) {
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
  if (p.alpha != 1.0f) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= p.alpha;
  }
  if (p.bias) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(bias_s + (h * 4 + g) * 4), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[g * 8 + e] += f[e];
    }
  }
  uint8_t* row_aux = buf_aux + lane * 128;
  uint8_t* row_c = buf_c + lane * 128;
  if (p.aux_out && p.act != 5) {
#pragma unroll
    for (int g = 0; g < 4; ++g)
      *reinterpret_cast<uint4*>(row_aux + (((h * 4 + g) ^ (lane & 7)) << 4)) =
          pack8(reinterpret_cast<const float(&)[8]>(v[g * 8]));
  }
  if (p.act == 5) {
    // GELU and its derivative from one tanh, on pairs of values; the derivative goes to the auxiliary block:
    //   y = x (0.5 + 0.5 t),  d = 0.5 + 0.5 (t + x (c0 + c2 x^2) (1 - t^2)),  t = tanh(x (c0 + c1 x^2))
    const f32x2 c0 = f2_splat(0.7978845608f), c1 = f2_splat(0.0356774081f), c2 = f2_splat(0.1070322243f);
    const f32x2 one = f2_splat(1.0f), hf = f2_splat(0.5f);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float d[8];
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        const int i = g * 8 + e;
        const f32x2 x = f2_pack(v[i], v[i + 1]);
        const f32x2 xx = f2_mul(x, x);
        float u0, u1;
        f2_unpack(f2_mul(x, f2_fma(xx, c1, c0)), u0, u1);
        const float t0 = tanh_fast(u0), t1 = tanh_fast(u1);
        const f32x2 t = f2_pack(t0, t1), nt = f2_pack(-t0, -t1);
        const f32x2 hx = f2_mul(x, hf);
        const f32x2 sl = f2_mul(x, f2_fma(xx, c2, c0));
        const f32x2 w = f2_fma(sl, f2_fma(nt, t, one), t);
        f2_unpack(f2_fma(w, hf, hf), d[e], d[e + 1]);
        f2_unpack(f2_fma(hx, t, hx), v[i], v[i + 1]);
      }
      *reinterpret_cast<uint4*>(row_aux + (((h * 4 + g) ^ (lane & 7)) << 4)) = pack8(d);
    }
  } else if (p.act == 2) {
    // GELU (tanh form) on pairs of values: x * (0.5 + 0.5 tanh(x (c0 + c1 x^2)))
    const f32x2 c0 = f2_splat(0.7978845608f), c1 = f2_splat(0.0356774081f), hf = f2_splat(0.5f);
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      const f32x2 x = f2_pack(v[i], v[i + 1]);
      const f32x2 u = f2_mul(x, f2_fma(f2_mul(x, x), c1, c0));
      float u0, u1;
      f2_unpack(u, u0, u1);
      const f32x2 t = f2_pack(tanh_fast(u0), tanh_fast(u1));
      const f32x2 hx = f2_mul(x, hf);
      f2_unpack(f2_fma(hx, t, hx), v[i], v[i + 1]);
    }
  } else if (p.act >= 1 && p.act <= 5) {
#pragma unroll
    for (int g = 0; g < 4; ++g) apply_act8(p.act, reinterpret_cast<float(&)[8]>(v[g * 8]));
  }
  if (in_kind) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float x[8];
      unpack8(*reinterpret_cast<const uint4*>(row_c + (((h * 4 + g) ^ (lane & 7)) << 4)), x);
      if (in_kind == 1) {
        if (p.act == 15) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[g * 8 + e] *= x[e];
        } else if (p.act == 12) {
          // GELU' on pairs: 0.5 (1 + t) + 0.5 x (1 - t^2) (c0 + c2 x^2),  t = tanh(x (c0 + c1 x^2))
          const f32x2 c0 = f2_splat(0.7978845608f), c1 = f2_splat(0.0356774081f), c2 = f2_splat(0.1070322243f);
          const f32x2 one = f2_splat(1.0f), hf = f2_splat(0.5f);
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            const f32x2 xp = f2_pack(x[e], x[e + 1]);
            const f32x2 xx = f2_mul(xp, xp);
            float u0, u1;
            f2_unpack(f2_mul(xp, f2_fma(xx, c1, c0)), u0, u1);
            const float t0 = tanh_fast(u0), t1 = tanh_fast(u1);
            const f32x2 t = f2_pack(t0, t1), nt = f2_pack(-t0, -t1);
            const f32x2 sl = f2_mul(xp, f2_fma(xx, c2, c0));
            const f32x2 w = f2_fma(sl, f2_fma(nt, t, one), t);          // t + sl (1 - t^2)
            const f32x2 d = f2_fma(w, hf, hf);                           // 0.5 + 0.5 w
            f2_unpack(f2_mul(f2_pack(v[g * 8 + e], v[g * 8 + e + 1]), d), v[g * 8 + e], v[g * 8 + e + 1]);
          }
        } else {
          apply_act_bwd8(p.act, reinterpret_cast<float(&)[8]>(v[g * 8]), x);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[g * 8 + e] += x[e];
      }
    }
  }
#pragma unroll
  for (int g = 0; g < 4; ++g)
    *reinterpret_cast<uint4*>(row_c + (((h * 4 + g) ^ (lane & 7)) << 4)) =
        pack8(reinterpret_cast<const float(&)[8]>(v[g * 8]));
}

// ----------------------------------------------------------------------------- all-reduce epilogue helpers
// Sum one 32 x 64 block over all ranks (fixed rank order), add bias / residual, write it to every rank's output.
__device__ __forceinline__ void ar_reduce_block(const GemmParams& p, long long blk_off, long long row0, long long col0,
                                                int lane) {
  const int rg = lane >> 3, cg = lane & 7;
  const long long col = col0 + cg * 8;
  if (col >= p.N) return;
  float bias8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (p.bias) {
#pragma unroll
    for (int e = 0; e < 8; ++e)
      bias8[e] = p.bias_f32 ? __ldg(static_cast<const float*>(p.bias) + col + e)
                            : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col + e]);
  }
  // Remote loads have microseconds of latency: all loads of a group of rows are issued before the first one is used
  // (8 rows at a time through the switch, 2 rows x all ranks at a time over peer pointers).
  auto finish = [&](int rl, float (&v)[8]) {
    const long long row = row0 + rl;
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] += bias8[e];
    // Reduce-scatter: the shard's buffers start at the shard's first row.
    const long long orow = p.ar.mode == 1 ? row - (long long)p.ar.rank * p.ar.rows_per_rank : row;
    if (p.residual) {
      float t[8];
      unpack8(*reinterpret_cast<const uint4*>(p.residual + orow * p.ldr + col), t);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += t[e];
    }
    const uint4 o = pack8(v);
    const long long o_off = orow * p.ldc + col;
    if (p.ar.mode == 1) {
      *reinterpret_cast<uint4*>(p.ar.out_peer[p.ar.rank] + o_off) = o;
    } else if (p.ar.use_nvls) {
      multimem_st_bf16x8(p.ar.mc_out + o_off, o);
    } else {
      for (int r = 0; r < p.ar.world; ++r) st_cg_v4(p.ar.out_peer[r] + o_off, o);
    }
  };
  if (p.ar.use_nvls) {
    uint4 raw[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int rl = it * 4 + rg;
      raw[it] = make_uint4(0, 0, 0, 0);
      if (row0 + rl < p.M) raw[it] = multimem_ld_reduce_bf16x8(p.ar.mc_partial + blk_off + rl * 64 + cg * 8);
    }
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int rl = it * 4 + rg;
      if (row0 + rl >= p.M) continue;
      float v[8];
      unpack8(raw[it], v);
      finish(rl, v);
    }
  } else {
#pragma unroll 1
    for (int it0 = 0; it0 < 8; it0 += 2) {
      uint4 raw[2][kMaxRanks];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int rl = (it0 + j) * 4 + rg;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
          raw[j][r] = make_uint4(0, 0, 0, 0);
          if (r < p.ar.world && row0 + rl < p.M) raw[j][r] = ld_cg_v4(p.ar.peer_partial[r] + blk_off + rl * 64 + cg * 8);
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int rl = (it0 + j) * 4 + rg;
        if (row0 + rl >= p.M) continue;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {   // fixed rank order; absent ranks contribute zeros
          float t[8];
          unpack8(raw[j][r], t);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] += t[e];
        }
        finish(rl, v);
      }
    }
  }
}

// ----------------------------------------------------------------------------- tensor-core kernel
constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kEpiWarps = 8;
constexpr int kGemmThreads = 32 * (2 + kEpiWarps);

// BROWS: rows (K-major) or columns (MN-major) of B one CTA stages: BN, or BN / 2 when a CTA pair shares the tile.
// EPI_BLOCKS: 4 KB staging blocks per epilogue warp (two for the tile-store epilogue, which keeps one store in flight).
template <int BN, int STAGES, int BROWS = BN, int EPI_BLOCKS = 1>
struct GemmSmem {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BROWS * kBK * 2;
  static constexpr int kStagePerWarp = EPI_BLOCKS * 4096;
  static constexpr int kStageOff = STAGES * (kABytes + kBBytes);   // epilogue staging
  static constexpr int kBiasOff = kStageOff + kEpiWarps * kStagePerWarp;   // 64 bf16 bias values per epilogue warp
  static constexpr int kBarOffset = kBiasOff + kEpiWarps * 128;
  // barriers: full / empty per stage, 2 + 2 accumulator, 1 drain, 2 epilogue-input per epilogue warp
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 4 + 1 + 2 * kEpiWarps) * 8 + 32 + 1024;  // + alignment slack
  static_assert(kTotal <= 227 * 1024, "GEMM: shared memory budget");
};

// Extra kernel parameter of the all-gather variant: one tensor map per rank's shard of A.
struct NoPeerMaps {};
template <bool AG> struct PeerMaps { using type = NoPeerMaps; };
template <> struct PeerMaps<true> { using type = TmapSet; };

// PAIR: the kernel is launched as clusters of two CTAs that share 256-row tiles (cta_group::2): CTA r of a pair stages
// rows [128 r, 128 r + 128) of the A tile and columns [BN/2 r, BN/2 r + BN/2) of the B tile, the leader's (r = 0)
// issuer thread runs the MMAs of both tensor cores, each CTA's epilogue warps drain their own 128 x BN accumulator.
// Work units are then pairs of row tiles; `tile` below stays the index of this CTA's own 128-row tile.
template <bool A_MN, bool B_MN, int BN, int STAGES, bool AG = false, bool PAIR = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ typename PeerMaps<AG>::type peers, const __grid_constant__ EpiMaps em,
               const GemmParams p) {
  static_assert(!(PAIR && AG), "the all-gather prologue runs on single CTAs");
  constexpr int BROWS = PAIR ? BN / 2 : BN;
  using L = GemmSmem<BN, STAGES, BROWS, PAIR ? 2 : 1>;
  constexpr int TMEM_COLS = 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * L::kABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* drain_bar = tmem_empty + 2;
  uint64_t* epi_in_bar = drain_bar + 1;            // [kEpiWarps][2]: an input block of the tile-store epilogue has landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(epi_in_bar + 2 * kEpiWarps);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* epi_ctr = reinterpret_cast<int*>(tmem_slot + 2);       // arrival counter of the epilogue-warp barrier
  volatile int* epi_last = reinterpret_cast<volatile int*>(tmem_slot + 3);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = PAIR ? cluster_cta_rank() : 0u;
  // Row tiles are handed out singly, or in pairs (the last pair of an odd count has a second half without rows: that
  // CTA stages zeros and its epilogue writes nothing).
  const int sched_tiles_m = PAIR ? (p.tiles_m + 1) / 2 : p.tiles_m;
  const int num_tiles = sched_tiles_m * p.tiles_n;
  const int num_units = num_tiles * p.splits;
  const int unit0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int unit_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  // Launch number of the all-reduce protocol; the word is rewritten only by the last CTA to leave.
  const uint32_t ar_epoch = p.ar.world > 0 ? *reinterpret_cast<volatile uint32_t*>(p.ar.epoch) + 1u : 0u;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *epi_ctr = 0;
    *epi_last = 0;
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    if (lane == 0) {
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(&full_bar[s], 1);
        mbar_init(&empty_bar[s], 1);
      }
      for (int a = 0; a < 2; ++a) {
        mbar_init(&tmem_full[a], 1);
        mbar_init(&tmem_empty[a], PAIR ? 2 * kEpiWarps : kEpiWarps);   // the leader's is released by both CTAs
      }
      mbar_init(drain_bar, 1);
      for (int w = 0; w < 2 * kEpiWarps; ++w) mbar_init(&epi_in_bar[w], 1);
      mbar_fence_init();
    }
    __syncwarp();
    if constexpr (PAIR) tmem_alloc_pair<TMEM_COLS>(tmem_slot);
    else tmem_alloc<TMEM_COLS>(tmem_slot);
  }
  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all();   // both CTAs' barriers exist before either signals the other's
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t issued = 0;
      uint32_t ag_ready_mask = 0;
      const uint32_t ag_epoch = AG ? *reinterpret_cast<const volatile uint32_t*>(p.ag.epoch) : 0u;
      (void)ag_ready_mask;
      (void)ag_epoch;
      DPTB_PROF_DECL(prof_wait);
      DPTB_PROF_BEGIN(prof_t_all);
      // Pair: both CTAs' copies count on the LEADER's full barrier (it expects the bytes of both).
      uint32_t full_addr[STAGES];
#pragma unroll
      for (int s = 0; s < STAGES; ++s) full_addr[s] = PAIR ? map_to_cta(&full_bar[s], 0) : smem_u32(&full_bar[s]);
      for (int unit = unit0; unit < num_units && !*abort_flag; unit += unit_step) {
        const int stile = unit % num_tiles;
        const int kb0 = (unit / num_tiles) * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        const int mi = PAIR ? (stile % sched_tiles_m) * 2 + (int)cta_rank : tile_row_index(p, stile);
        const int m0 = mi * kBM;
        const int n0 = (stile / sched_tiles_m) * BN + (PAIR ? (int)cta_rank * BROWS : 0);
        const CUtensorMap* a_map = &tmA;
        int a_row = m0;
        if constexpr (AG) {
          // Rows of another rank: wait (once per source, bounded) until its shard is published, then read it in place.
          const int src = mi / p.ag.tiles_per_rank;
          a_map = &peers.m[src];
          a_row = (mi % p.ag.tiles_per_rank) * kBM;
          if (!((ag_ready_mask >> src) & 1u)) {
            if (src != p.ag.rank && !wait_flag_ge(p.ag.ready + src, ag_epoch)) {
              *abort_flag = 1;
              break;
            }
            asm volatile("fence.proxy.async;" ::: "memory");   // the flag was read by the generic proxy, the tiles are not
            ag_ready_mask |= 1u << src;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb, ++issued) {
          const int s = issued % STAGES;
          const uint32_t ph = (issued / STAGES) & 1;
          DPTB_PROF_BEGIN(prof_t0);
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, kWaitEmptyTimeout)) break;
          DPTB_PROF_END(prof_t0, prof_wait);
          uint8_t* a_dst = sA + s * L::kABytes;
          uint8_t* b_dst = sB + s * L::kBBytes;
          if constexpr (PAIR) {
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * (L::kABytes + L::kBBytes));
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < kBM / 64; ++j)
                tma_load_2d_pair(a_dst + j * 8192, &tmA, full_addr[s], m0 + j * 64, kb * kBK);
            } else {
              tma_load_2d_pair(a_dst, &tmA, full_addr[s], kb * kBK, m0);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BROWS / 64; ++j)
                tma_load_2d_pair(b_dst + j * 8192, &tmB, full_addr[s], n0 + j * 64, kb * kBK);
            } else {
              tma_load_2d_pair(b_dst, &tmB, full_addr[s], kb * kBK, n0);
            }
          } else {
            mbar_arrive_expect_tx(&full_bar[s], L::kABytes + L::kBBytes);
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < kBM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, &full_bar[s], m0 + j * 64, kb * kBK);
            } else {
              tma_load_2d(a_dst, a_map, &full_bar[s], kb * kBK, a_row);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, &full_bar[s], n0 + j * 64, kb * kBK);
            } else {
              tma_load_2d(b_dst, &tmB, &full_bar[s], kb * kBK, n0);
            }
          }
        }
      }
      DPTB_PROF_STORE(0, prof_wait);
      DPTB_PROF_STORE(1, clock64() - prof_t_all);
      if (PAIR && *abort_flag && cta_rank != 0) {
        // The second CTA's copies are counted on the leader's barriers, which it cannot poll: give copies in flight
        // (microseconds) time to land before this CTA may leave.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
      } else if (*abort_flag) {
        // Do not leave while a tile copy may still be writing this CTA's shared memory.
        const uint32_t n = issued < (uint32_t)STAGES ? issued : (uint32_t)STAGES;
        for (uint32_t j = 0; j < n; ++j) {
          const uint32_t i = issued - 1 - j;
          uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(&full_bar[i % STAGES], (i / STAGES) & 1)) {
            if (global_timer_ns() - t0 > kWaitLimitNs / 4) {
              report_error(kWaitDrainTimeout);
              break;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(PAIR ? 2 * kBM : kBM, BN, A_MN, B_MN);
      // Pair: a completion is signalled to the same barrier of both CTAs by one commit.
      uint32_t consumed = 0;
      uint32_t local_tile = 0;
      bool issued_any = false;
      DPTB_PROF_DECL(prof_wait_full);
      DPTB_PROF_DECL(prof_wait_acc);
      DPTB_PROF_BEGIN(prof_t_all);
      for (int unit = unit0; unit < num_units && !*abort_flag; unit += unit_step, ++local_tile) {
        const int kb0 = (unit / num_tiles) * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        DPTB_PROF_BEGIN(prof_t1);
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag, kWaitTmemEmptyTimeout)) break;
        DPTB_PROF_END(prof_t1, prof_wait_acc);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb, ++consumed) {
          const int s = consumed % STAGES;
          const uint32_t ph = (consumed / STAGES) & 1;
          DPTB_PROF_BEGIN(prof_t0);
          if (!mbar_wait(&full_bar[s], ph, abort_flag, kWaitFullTimeout)) { ok = false; break; }
          DPTB_PROF_END(prof_t0, prof_wait_full);
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + s * L::kABytes);
          const uint32_t b_addr = smem_u32(sB + s * L::kBBytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(a_addr + k * 2048, 8192, 1024) : make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(b_addr + k * 2048, 8192, 1024) : make_smem_desc(b_addr + k * 32, 16, 1024);
            if constexpr (PAIR) umma_bf16_pair(d_tmem, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
            else umma_bf16(d_tmem, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          issued_any = true;
          if constexpr (PAIR) {       // stage reusable (in both CTAs) once these MMAs have read it
            umma_commit_pair_both(&empty_bar[s]);
          } else {
            umma_commit(&empty_bar[s]);
          }
        }
        if (!ok) break;
        if constexpr (PAIR) {         // accumulator complete (each CTA's half)
          umma_commit_pair_both(&tmem_full[acc]);
        } else {
          umma_commit(&tmem_full[acc]);
        }
      }
      DPTB_PROF_STORE(2, prof_wait_full);
      DPTB_PROF_STORE(3, prof_wait_acc);
      DPTB_PROF_STORE(4, clock64() - prof_t_all);
      DPTB_PROF_STORE(7, local_tile);
      if (*abort_flag && issued_any) {
        if constexpr (PAIR) umma_commit_pair(smem_u32(drain_bar));
        else umma_commit(drain_bar);
        uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(drain_bar, 0)) {
          if (global_timer_ns() - t0 > kWaitLimitNs / 4) {
            report_error(kWaitDrainTimeout);
            break;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (two per TMEM lane quarter)
    const int ew = warp - 2;
    const int q = warp & 3;      // TMEM lane quarter this warp may read
    const int half = ew >> 2;    // takes the 64-column chunks with this parity
    uint8_t* stage = smem + L::kStageOff + ew * L::kStagePerWarp;
    uint32_t local_tile = 0;
    uint32_t epi_blk = 0;        // blocks this warp has stored through the tile-store epilogue
    uint32_t epi_in_ph = 0;      // phases of this warp's two input barriers (bit j: staging block j)
    uint32_t epi_in_pf = 0;      // bit j: the input of the coming tile's block j has been requested already
    int epi_gen = 0;
    // Registers of one 64-column chunk of this thread's row -> final epilogue (staged bf16 path or direct fp32 path).
    auto emit = [&](long long row0, long long col0, const uint32_t (&r0)[32], const uint32_t (&r1)[32]) {
      if (p.out_f32) {
        if (row0 + lane < p.M) {
          epilogue_direct_f32(p, row0 + lane, col0, r0);
          if (col0 + 32 < p.N) epilogue_direct_f32(p, row0 + lane, col0 + 32, r1);
        }
      } else {
        uint8_t* srow = stage + lane * 128;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint32_t* src = g < 4 ? &r0[g * 8] : &r1[(g - 4) * 8];
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(src[0]) * p.alpha, __uint_as_float(src[1]) * p.alpha);
          u.y = pack_bf16x2(__uint_as_float(src[2]) * p.alpha, __uint_as_float(src[3]) * p.alpha);
          u.z = pack_bf16x2(__uint_as_float(src[4]) * p.alpha, __uint_as_float(src[5]) * p.alpha);
          u.w = pack_bf16x2(__uint_as_float(src[6]) * p.alpha, __uint_as_float(src[7]) * p.alpha);
          *reinterpret_cast<uint4*>(srow + ((g ^ (lane & 7)) << 4)) = u;
        }
        __syncwarp();
        epilogue_phase2(p, stage, row0, col0, lane);
        __syncwarp();
      }
    };
    uint32_t* bias_s = reinterpret_cast<uint32_t*>(smem + L::kBiasOff) + ew * 32;
    // Tiles this rank owns whose cross-rank reduction is still outstanding (all-reduce epilogue).
    int ar_tile[2] = {0, 0};
    int ar_pending = 0;
    auto ar_reduce_tile = [&](int t) -> bool {
      bool got = true;
      if (lane < p.ar.world) got = wait_flag_ge(p.ar.flags_peer[p.ar.rank] + (size_t)t * kMaxRanks + lane, ar_epoch);
      if (!__all_sync(0xffffffffu, got)) {
        *abort_flag = 1;
        return false;
      }
      const int tm0 = tile_row_index(p, t) * kBM;
      const int tn0 = (t / p.tiles_m) * BN;
#pragma unroll 1
      for (int c = half; c < BN / 64; c += 2) {
        const long long col0 = (long long)tn0 + c * 64;
        if (col0 >= p.N) break;
        ar_reduce_block(p, (long long)t * (BN * kBM) + (long long)c * (64 * kBM) + (long long)(q * 32) * 64,
                        (long long)tm0 + q * 32, col0, lane);
      }
      return true;
    };
    // Bounded barrier over the epilogue warps (a hardware named barrier could not give up).
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      epi_gen += kEpiWarps;
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
    DPTB_PROF_DECL(prof_wait_acc);
    DPTB_PROF_DECL(prof_ld);
    DPTB_PROF_DECL(prof_fin);
    DPTB_PROF_DECL(prof_blocks);
    DPTB_PROF_BEGIN(prof_t_all);
    // The accumulator is handed back to the issuer: in a pair, to the leader's barrier, by both CTAs.
    const uint32_t tmem_empty_addr[2] = {PAIR ? map_to_cta(&tmem_empty[0], 0) : 0u,
                                         PAIR ? map_to_cta(&tmem_empty[1], 0) : 0u};
    auto release_acc = [&](uint32_t acc) {
      if constexpr (PAIR) mbar_arrive_cluster(tmem_empty_addr[acc]);
      else mbar_arrive(&tmem_empty[acc]);
    };
    for (int unit = unit0; unit < num_units && !*abort_flag; unit += unit_step, ++local_tile) {
      const int stile = unit % num_tiles;
      const int split = unit / num_tiles;
      const int mi = PAIR ? (stile % sched_tiles_m) * 2 + (int)cta_rank : tile_row_index(p, stile);
      const int ni = stile / sched_tiles_m;
      const int tile = PAIR ? ni * p.tiles_m + mi : stile;   // this CTA's own 128-row tile (workspace / counter index)
      const int m0 = mi * kBM;
      const int n0 = ni * BN;
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      // Tile-store epilogue: this warp's bias slices are requested before the wait for the accumulator, and the
      // per-element input blocks (residual / saved activation derivative / C) are fetched into the staging blocks by
      // tile loads one block of work ahead: block 0 of a tile while block 1 of the tile before it is worked on, block 1
      // here, while block 0 is worked on.  Neither latency is paid after the accumulator has arrived.
      uint32_t bias_pf[BN / 128] = {};
      const int epi_in_kind = p.act >= 11 ? 1 : (p.residual ? 2 : (p.accumulate ? 3 : 0));
      if constexpr (PAIR) {
        if (p.row_epi == 3 && p.splits == 1 && mi < p.tiles_m && (long long)m0 + q * 32 < p.M) {
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) {
              const long long col = (long long)n0 + (half + 2 * j) * 64 + 2 * lane;
              if (col < p.N)
                bias_pf[j] = __ldg(reinterpret_cast<const uint32_t*>(static_cast<const __nv_bfloat16*>(p.bias) + col));
            }
          }
          if (epi_in_kind) {
            // Block 0 when it was not requested during the previous tile (the first tile of this CTA, or one that
            // follows a tile without rows): wait until the stores have finished reading the staging block, then load.
            if (!(epi_in_pf & 1u) && (long long)n0 + half * 64 < p.N && lane == 0) {
              bulk_wait_read_all();
              mbar_arrive_expect_tx(&epi_in_bar[ew * 2], 4096u);
              tma_load_2d(stage, &em.in, &epi_in_bar[ew * 2], n0 + half * 64, m0 + q * 32);
            }
          }
        }
        epi_in_pf = 0;
      }
      DPTB_PROF_BEGIN(prof_t0);
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[acc], acc_ph, abort_flag, kWaitTmemFullTimeout))) break;
      DPTB_PROF_END(prof_t0, prof_wait_acc);
      tc_fence_after_sync();
      if (PAIR && mi >= p.tiles_m) {   // second half of the last, odd pair: no rows to write
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) release_acc(acc);
        continue;
      }
      const long long row0 = (long long)m0 + q * 32;
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      if (!PAIR && p.ar.world > 0) {
        // Partial tile -> this rank's partial buffer (each thread writes its row's 128 bytes of a 64-column block as
        // whole sectors); flag the owner.  The CTA-wide barrier orders every warp's stores before the one
        // release-at-system-scope store of the flag (release is cumulative over that synchronisation).
        __nv_bfloat16* ptile = p.ar.partial + (size_t)tile * (BN * kBM);
#pragma unroll 1
        for (int c = half; c < BN / 64; c += 2) {
          if ((long long)n0 + c * 64 >= p.N) break;  // warp-uniform
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_row + c * 64, r0);
          tmem_ld_32x32(t_row + c * 64 + 32, r1);
          tmem_ld_wait();
          uint4 o[8];
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const uint32_t* src = g < 4 ? &r0[g * 8] : &r1[(g - 4) * 8];
            o[g].x = pack_bf16x2(__uint_as_float(src[0]) * p.alpha, __uint_as_float(src[1]) * p.alpha);
            o[g].y = pack_bf16x2(__uint_as_float(src[2]) * p.alpha, __uint_as_float(src[3]) * p.alpha);
            o[g].z = pack_bf16x2(__uint_as_float(src[4]) * p.alpha, __uint_as_float(src[5]) * p.alpha);
            o[g].w = pack_bf16x2(__uint_as_float(src[6]) * p.alpha, __uint_as_float(src[7]) * p.alpha);
          }
          if (row0 + lane < p.M)
            st_row64(ptile + (size_t)c * (64 * kBM) + (size_t)(q * 32 + lane) * 64, true, o);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) release_acc(acc);   // the issuer may start the next tile in this accumulator
        if (!epi_sync()) break;                          // every epilogue warp has written its blocks
        const int owner = p.ar.mode == 1 ? m0 / p.ar.rows_per_rank : tile % p.ar.world;
        if (ew == 0 && lane == 0)
          st_release_sys(p.ar.flags_peer[owner] + (size_t)tile * kMaxRanks + p.ar.rank, ar_epoch);
        // The owner's reduction of a tile is deferred until two more tiles have been stored: by then the other
        // ranks' partials of that tile have usually arrived, so the wait does not stall the pipeline.
        if (owner == p.ar.rank) {
          if (ar_pending == 2) {
            if (!ar_reduce_tile(ar_tile[0])) break;
            ar_tile[0] = ar_tile[1];
            ar_pending = 1;
          }
          ar_tile[ar_pending++] = tile;
        }
      } else if (PAIR && p.splits == 1) {   // pairs are launched only for outputs this epilogue can take
        // Tile-store epilogue: registers -> swizzled staging block -> one tile store per 32 x 64 block, with the
        // per-element input (if any) fetched into the same block by a tile load while the accumulator is read.
        const int in_kind = epi_in_kind;
        const bool rows_live = row0 < p.M;   // warp-uniform
        bool ok = true;
#pragma unroll 1
        for (int j = 0; j < BN / 128 && ok; ++j) {
          const int c = half + 2 * j;
          const long long col0 = (long long)n0 + c * 64;
          if (col0 >= p.N || !rows_live) break;  // warp-uniform
          // Staging block of the output: with an input, the block the input of this chunk was loaded into; with a
          // pre-activation copy, block 1 (block 0 stages the copy); else the two blocks alternate.
          uint8_t* buf_aux = stage;
          uint8_t* buf_c = stage + (in_kind ? j * 4096 : (p.aux_out ? 4096 : (int)(epi_blk & 1) * 4096));
          DPTB_PROF_BEGIN(prof_c0);
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_row + c * 64, r0);
          tmem_ld_32x32(t_row + c * 64 + 32, r1);
          if (p.bias) bias_s[lane] = bias_pf[j];
          if (!in_kind && lane == 0) {
            // the stores that last read the block(s) about to be overwritten have finished reading
            if (p.aux_out) bulk_wait_read_all();
            else bulk_wait_read_1();
          }
          if (in_kind) {
            if (BN / 128 > 1 && j == 0 && col0 + 128 < p.N) {
              // Block 1's input, while the accumulator load above is in flight: its staging block was handed to a
              // store at the end of the previous tile, which has had the accumulator wait to finish reading it.
              if (lane == 0) {
                bulk_wait_read_all();
                mbar_arrive_expect_tx(&epi_in_bar[ew * 2 + 1], 4096u);
                tma_load_2d(stage + 4096, &em.in, &epi_in_bar[ew * 2 + 1], (int)col0 + 128, (int)row0);
              }
            }
            if (BN / 128 > 1 && j == BN / 128 - 1 && unit + unit_step < num_units) {
              // The first block of the NEXT tile is requested now, a block's worth of work before it is needed: its
              // staging block is free once this tile's first store has finished reading it.
              const int ns = (unit + unit_step) % num_tiles;
              const int nmi = (ns % sched_tiles_m) * 2 + (int)cta_rank;
              const int nx_m0 = nmi * kBM, nx_n0 = (ns / sched_tiles_m) * BN;
              if (nmi < p.tiles_m && (long long)nx_m0 + q * 32 < p.M && (long long)nx_n0 + half * 64 < p.N) {
                if (lane == 0) {
                  bulk_wait_read_all();
                  mbar_arrive_expect_tx(&epi_in_bar[ew * 2], 4096u);
                  tma_load_2d(stage, &em.in, &epi_in_bar[ew * 2], nx_n0 + half * 64, nx_m0 + q * 32);
                }
                epi_in_pf |= 1u;
              }
            }
            ok = __all_sync(0xffffffffu, mbar_wait(&epi_in_bar[ew * 2 + j], (epi_in_ph >> j) & 1u, abort_flag,
                                                   kWaitFullTimeout));
            epi_in_ph ^= 1u << j;
          }
          tmem_ld_wait();
          __syncwarp();              // bias slice and buffer release are visible to every lane
          if (!ok) break;
          DPTB_PROF_END(prof_c0, prof_ld);
          DPTB_PROF_BEGIN(prof_c1);
          epi_half_tma(p, bias_s, 0, lane, in_kind, r0, buf_aux, buf_c);
          epi_half_tma(p, bias_s, 1, lane, in_kind, r1, buf_aux, buf_c);
          fence_proxy_async_smem();
          __syncwarp();              // also: every lane has read the bias slice before the next block rewrites it
          if (lane == 0) {
            if (p.aux_out) {
              tma_store_2d(&em.aux, buf_aux, (int)col0, (int)row0);
              bulk_commit_group();
            }
            tma_store_2d(&em.c, buf_c, (int)col0, (int)row0);
            bulk_commit_group();
          }
          DPTB_PROF_END(prof_c1, prof_fin);
          ++epi_blk;
#ifdef DPTB_GEMM_PROFILE
          ++prof_blocks;
#endif
        }
        if (!ok) break;
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) release_acc(acc);
      } else if (!PAIR && p.splits == 1) {
#pragma unroll 1
        for (int c = half; c < BN / 64; c += 2) {
          const long long col0 = (long long)n0 + c * 64;
          if (col0 >= p.N) break;  // warp-uniform
          uint32_t r0[32], r1[32];
          DPTB_PROF_BEGIN(prof_c0);
          tmem_ld_32x32(t_row + c * 64, r0);
          tmem_ld_32x32(t_row + c * 64 + 32, r1);
          if (p.row_epi && col0 + 64 <= p.N) {
            EpiIn in;
            epi_prefetch(p, bias_s, row0 + lane, col0, lane, in);
            tmem_ld_wait();
            DPTB_PROF_END(prof_c0, prof_ld);
            DPTB_PROF_BEGIN(prof_c1);
            epi_finish_row(p, bias_s, row0, col0, lane, r0, r1, in);
            DPTB_PROF_END(prof_c1, prof_fin);
          } else {
            tmem_ld_wait();
            DPTB_PROF_END(prof_c0, prof_ld);
            DPTB_PROF_BEGIN(prof_c1);
            emit(row0, col0, r0, r1);
            DPTB_PROF_END(prof_c1, prof_fin);
          }
#ifdef DPTB_GEMM_PROFILE
          ++prof_blocks;
#endif
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) release_acc(acc);
      } else {
        // Partial accumulator -> workspace, column-major inside the tile so that a warp writes 128 contiguous bytes.
        float* wtile = p.ws + (size_t)tile * p.splits * (BN * kBM);
        float* wmine = wtile + (size_t)split * (BN * kBM) + q * 32 + lane;
#pragma unroll 1
        for (int c = half; c < BN / 64; c += 2) {
          if ((long long)n0 + c * 64 >= p.N) break;
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_row + c * 64, r0);
          tmem_ld_32x32(t_row + c * 64 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            wmine[(c * 64 + i) * kBM] = __uint_as_float(r0[i]);
            wmine[(c * 64 + 32 + i) * kBM] = __uint_as_float(r1[i]);
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) release_acc(acc);
        __threadfence();
        if (!epi_sync()) break;
        if (ew == 0 && lane == 0) {
          const int old = atomicAdd(&p.counters[tile], 1);
          const int last = old == p.splits - 1;
          if (last) p.counters[tile] = 0;  // ready for the next launch
          *epi_last = last;
        }
        if (!epi_sync()) break;
        const bool last = *epi_last != 0;
        if (last) {
          __threadfence();
          const float* wrow = wtile + q * 32 + lane;
#pragma unroll 1
          for (int c = half; c < BN / 64; c += 2) {
            const long long col0 = (long long)n0 + c * 64;
            if (col0 >= p.N) break;
            uint32_t r0[32], r1[32];
            const bool tma = p.row_epi && col0 + 64 <= p.N;
            EpiIn in;
            if (tma) epi_prefetch(p, bias_s, row0 + lane, col0, lane, in);
            // Split index outermost: the 32 loads of one split are independent and stay in flight together; the
            // additions still happen in split order for every element.
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              float acc32[32];
#pragma unroll
              for (int i = 0; i < 32; ++i) acc32[i] = 0.0f;
              for (int sp = 0; sp < p.splits; ++sp) {
                const float* src = wrow + (size_t)sp * (BN * kBM) + (size_t)(c * 64 + hh * 32) * kBM;
#pragma unroll
                for (int i = 0; i < 32; ++i) acc32[i] += __ldcg(src + i * kBM);
              }
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (hh == 0) r0[i] = __float_as_uint(acc32[i]);
                else r1[i] = __float_as_uint(acc32[i]);
              }
            }
            if (tma) epi_finish_row(p, bias_s, row0, col0, lane, r0, r1, in);
            else emit(row0, col0, r0, r1);
          }
        }
        if (!epi_sync()) break;  // epi_last may be rewritten only after every warp has read it
      }
    }
    if constexpr (!PAIR) {
      for (int i = 0; i < ar_pending && !*abort_flag; ++i)
        if (!ar_reduce_tile(ar_tile[i])) break;
    }
    if (PAIR && lane == 0) bulk_wait_read_all();   // tile stores of this warp have finished reading its staging blocks
#ifdef DPTB_GEMM_PROFILE
    if (ew == 0 && lane == 0) {
      DPTB_PROF_STORE(5, prof_wait_acc);
      DPTB_PROF_STORE(6, clock64() - prof_t_all);
      DPTB_PROF_STORE(8, prof_ld);
      DPTB_PROF_STORE(9, prof_fin);
      DPTB_PROF_STORE(10, prof_blocks);
    }
#endif
  }

  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all();   // neither CTA leaves while the other may still signal its barriers
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (PAIR) tmem_dealloc_pair<TMEM_COLS>(tmem_base);
    else tmem_dealloc<TMEM_COLS>(tmem_base);
  }
  if (!PAIR && p.ar.world > 0 && threadIdx.x == 0) {
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

// ----------------------------------------------------------------------------- SIMT fallback
// Any shape, any stride, fp32 or bf16 inputs.  64x64 tile, 16x16 threads, 4x4 outputs per thread.
template <typename TA, typename TB>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, long long sam, long long sak, const TB* __restrict__ B, long long sbk,
                 long long sbn, const GemmParams p) {
  __shared__ float As[16][64 + 1];
  __shared__ float Bs[16][64 + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const long long m0 = (long long)blockIdx.y * 64, n0 = (long long)blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < p.K; k0 += 16) {
    for (int i = threadIdx.x; i < 16 * 64; i += 256) {
      const int kk = i & 15, mm = i >> 4;
      const long long m = m0 + mm, n = n0 + mm, k = k0 + kk;
      As[kk][mm] = (m < p.M && k < p.K) ? (float)A[m * sam + k * sak] : 0.0f;
      Bs[kk][mm] = (n < p.N && k < p.K) ? (float)B[k * sbk + n * sbn] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      const long long m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < p.M && n < p.N) epilogue_scalar(p, m, n, acc[i][j]);
    }
}

template <bool A_MN, bool B_MN, int BN, int STAGES>
static int launch_tc(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES>;
  auto kern = gemm_tc_kernel<A_MN, B_MN, BN, STAGES>;
  static bool configured = false;
  if (!configured) {
    DPTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    configured = true;
  }
  const int tiles = p.tiles_m * p.tiles_n * p.splits;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kGemmThreads, L::kTotal, stream>>>(tmA, tmB, NoPeerMaps{}, EpiMaps{}, p);
  return counted(1, (int)cudaGetLastError());
}

// CTA-pair variant: clusters of two CTAs, one 256-row tile per pair (see the kernel's PAIR parameter).
constexpr int kPairStages256 = 5;   // 32 KB per stage and CTA, 64 KB of epilogue staging
constexpr int kPairStages128 = 6;   // 24 KB per stage and CTA
template <bool A_MN, bool B_MN, int BN, int STAGES>
static int pair_clusters(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr) {
  // Clusters of this kernel that can be resident at once (a persistent grid must not exceed it), once per process.
  using L = GemmSmem<BN, STAGES, BN / 2, 2>;
  auto kern = gemm_tc_kernel<A_MN, B_MN, BN, STAGES, false, true>;
  static int cached = -1;
  if (cached < 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return 0;
    cfg->gridDim = dim3(2 * (sm_count() / 2));
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 0;
    }
    cached = n;
    if (getenv("DPTB_GEMM_VERBOSE")) fprintf(stderr, "gemm pair BN=%d: %d clusters of 2 CTAs can be resident\n", BN, n);
  }
  (void)attr;
  return cached;
}
template <bool A_MN, bool B_MN, int BN, int STAGES>
static int launch_tc_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const EpiMaps& em, const GemmParams& p,
                          cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES, BN / 2, 2>;
  auto kern = gemm_tc_kernel<A_MN, B_MN, BN, STAGES, false, true>;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = L::kTotal;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int max_clusters = pair_clusters<A_MN, B_MN, BN, STAGES>(&cfg, attr);
  if (max_clusters <= 0) return kErrUnsupported;
  const int units = ((p.tiles_m + 1) / 2) * p.tiles_n * p.splits;
  const int clusters = units < max_clusters ? units : max_clusters;
  cfg.gridDim = dim3(2 * clusters);
  return counted(1, (int)cudaLaunchKernelEx(&cfg, kern, tmA, tmB, NoPeerMaps{}, em, p));
}

// All-gather variant: A (K-major) comes from every rank's shard, B is an nn.Linear weight (K-major).
template <int BN, int STAGES>
static int launch_tc_ag(const TmapSet& peers, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES>;
  auto kern = gemm_tc_kernel<false, false, BN, STAGES, true>;
  static bool configured = false;
  if (!configured) {
    DPTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    configured = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kGemmThreads, L::kTotal, stream>>>(peers.m[p.ag.rank], tmB, peers, EpiMaps{}, p);
  return counted(1, (int)cudaGetLastError());
}

}  // namespace dptb

using namespace dptb;

// Peer-memory description of the all-gather prologue (see TpAg): every rank's shard of A, [rows_per_rank, lda] each.
struct DptbTpAgArgs {
  int world, rank;
  long long rows_per_rank;
  const void* a_peer[kMaxRanks];
  const void* ready;   // local flag words [kMaxRanks], raised by dptb_tp_signal on the peers
  const void* epoch;   // local word written by this rank's dptb_tp_signal: the value the flags must have reached
};
// 32-bit words of a flag array for `max_tiles` tiles.
extern "C" long long dptb_tp_flag_words(int max_tiles) { return ((long long)max_tiles + 1) * kMaxRanks; }

static int gemm_impl(const DptbGemmArgs* a, const DptbTpArArgs* ar, const DptbTpAgArgs* ag, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (a->M <= 0 || a->N <= 0) return 0;
  if (a->K < 0) return kErrBadShape;
  GemmParams p;
  p.ar.world = 0;
  p.ar.mode = 0;
  p.ar.rows_per_rank = 0;
  p.ag.world = 0;
  const void* a_ptr = a->A;
  if (ag) {
    if (ar || ag->world < 1 || ag->world > kMaxRanks || ag->rank < 0 || ag->rank >= ag->world) return kErrBadShape;
    if (a->trans_a || !a->trans_b || ag->rows_per_rank <= 0 || ag->rows_per_rank % kBM ||
        ag->rows_per_rank * ag->world != a->M)
      return kErrBadShape;
    a_ptr = ag->a_peer[ag->rank];
  }
  p.M = a->M; p.N = a->N; p.K = a->K;
  p.C = a->C; p.ldc = a->ldc;
  p.bias = a->bias; p.bias_f32 = a->bias_f32;
  p.residual = static_cast<const __nv_bfloat16*>(a->residual); p.ldr = a->ldr;
  p.aux_out = static_cast<__nv_bfloat16*>(a->aux_out); p.ld_aux_out = a->ld_aux_out;
  p.aux_in = static_cast<const __nv_bfloat16*>(a->aux_in); p.ld_aux_in = a->ld_aux_in;
  p.act = a->act; p.out_f32 = a->out_f32; p.accumulate = a->accumulate; p.alpha = a->alpha;
  if (p.act >= 11 && !p.aux_in) return kErrBadShape;
  if (p.act == 5 && !p.aux_out) p.act = 2;

  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool tc_ok = !a->force_simt && !a->a_f32 && !a->b_f32 && a->K > 0 && al16(a_ptr) && al16(a->B) &&
                     (a->lda % 8 == 0) && (a->ldb % 8 == 0);
  p.vec_ok = al16(p.C) && (p.ldc % 8 == 0) && (!p.bias || al16(p.bias)) &&
             (!p.residual || (al16(p.residual) && p.ldr % 8 == 0)) &&
             (!p.aux_out || (al16(p.aux_out) && p.ld_aux_out % 8 == 0)) &&
             (!p.aux_in || (al16(p.aux_in) && p.ld_aux_in % 8 == 0));

  if (ar) {
    // The all-reduce epilogue exists on the tensor-core path only and moves whole 16-byte groups.
    if (!tc_ok || !p.vec_ok || (a->N % 8) || a->out_f32 || a->act || a->aux_out || a->aux_in || a->accumulate)
      return kErrUnsupported;
    if (ar->world < 1 || ar->world > kMaxRanks || ar->rank < 0 || ar->rank >= ar->world) return kErrBadShape;
    if (ar->mode == 1 && (a->M % (ar->world * kBM))) return kErrBadShape;   // whole row tiles per shard
  }
  if (ag && (!tc_ok || a->splits > 1)) return kErrUnsupported;
  if (!tc_ok) {
    p.tiles_m = p.tiles_n = p.num_kb = 0;
    p.splits = 1; p.kb_per_split = 0; p.ws = nullptr; p.counters = nullptr;
    dim3 grid((unsigned)((a->N + 63) / 64), (unsigned)((a->M + 63) / 64));
    const long long sam = a->trans_a ? 1 : a->lda, sak = a->trans_a ? a->lda : 1;
    const long long sbk = a->trans_b ? 1 : a->ldb, sbn = a->trans_b ? a->ldb : 1;
    if (a->a_f32 && a->b_f32)
      gemm_simt_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)a->A, sam, sak, (const float*)a->B, sbk, sbn, p);
    else if (!a->a_f32 && !a->b_f32)
      gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)a->A, sam, sak, (const __nv_bfloat16*)a->B, sbk, sbn, p);
    else if (a->a_f32)
      gemm_simt_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>((const float*)a->A, sam, sak, (const __nv_bfloat16*)a->B, sbk, sbn, p);
    else
      gemm_simt_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)a->A, sam, sak, (const float*)a->B, sbk, sbn, p);
    return counted(1, (int)cudaGetLastError());
  }

  // Tile width and split-K factor from a small cost model (unit: the time of one 128x256x64 k-block).
  //   a CTA runs ceil(units / SMs) units back to back; a unit costs its k-blocks (a 128-wide tile moves as many bytes
  //   for half the math, so its k-block counts 0.75) plus a fixed prologue/epilogue, plus the partial-tile round
  //   trip when K is split.
  const int num_kb = (a->K + kBK - 1) / kBK;
  const int tm = (a->M + kBM - 1) / kBM;
  // CTA pairs (256-row tiles shared by two SMs) for every plain GEMM with at least two row tiles; the fused
  // tensor-parallel variants keep single CTAs.  DPTB_GEMM_PAIR=0 switches pairs off (for comparisons).
  static const bool pairs_enabled = [] {
    const char* e = getenv("DPTB_GEMM_PAIR");
    return !(e && e[0] == '0');
  }();
  // A pair's epilogue leaves through tile stores: bf16 output, every per-element buffer describable by a tensor map
  // (16-byte aligned, strides multiples of 16 bytes), at most one per-element input, and a pre-activation copy not
  // combined with an input (a warp's two staging blocks cover either case).
  const int epi_inputs = (p.act >= 11 ? 1 : 0) + (p.residual ? 1 : 0) + (p.accumulate ? 1 : 0);
  const bool tile_store_ok = !p.out_f32 && p.vec_ok && !(p.bias && p.bias_f32) && (a->N % 8) == 0 && epi_inputs <= 1 &&
                             !(epi_inputs == 1 && p.aux_out);
  const bool pair = pairs_enabled && !ar && !ag && tm >= 2 && tile_store_ok;
  // Work units run on `sms` CTAs, or on sms / 2 pairs, each pair taking two row tiles at a time.
  const int sms = pair ? sm_count() / 2 : sm_count();
  const int tm_sched = pair ? (tm + 1) / 2 : tm;
  int bn = a->bn, splits = a->splits;
  {
    double best = 1e30;
    int best_bn = 128, best_sp = 1;
    for (int cand_bn = 128; cand_bn <= 256; cand_bn += 128) {
      if (a->bn == 128 || a->bn == 256) { if (cand_bn != a->bn) continue; }
      if (cand_bn == 256 && a->N <= 128) continue;
      const int tiles = tm * ((a->N + cand_bn - 1) / cand_bn);
      const int sched_tiles = tm_sched * ((a->N + cand_bn - 1) / cand_bn);
      for (int sp = 1; sp <= 8; ++sp) {
        if (a->splits >= 1 && sp != a->splits) continue;
        if ((ar || ag) && sp > 1) break;
        if (sp > 1) {
          if (!a->ws || !a->counters || tiles > a->num_counters) break;
          if ((long long)tiles * sp * cand_bn * kBM * 4 > a->ws_bytes) break;
          if (num_kb / sp < 4) break;
        }
        const int kbs = (num_kb + sp - 1) / sp;
        const long long units = (long long)sched_tiles * sp;
        const double waves = (double)((units + sms - 1) / sms);
        const double per_kb = cand_bn == 256 ? 1.0 : 0.75;
        // (the fold of a 256-wide tile is serial in its last CTA: measured on 768 x 768 x 16384, 8 splits of 256-wide tiles
        // took 48 us against 42 us for 4 splits of 128-wide ones)
        const double fixed = (cand_bn == 256 ? 8.0 : 5.0) + (sp > 1 ? (cand_bn == 256 ? 8.0 + 2.5 * sp : 4.0 + 1.0 * sp) : 0.0);
        const double cost = waves * (kbs * per_kb + fixed);
        if (cost < best) { best = cost; best_bn = cand_bn; best_sp = sp; }
      }
    }
    bn = best_bn;
    splits = best_sp;
  }
  p.tiles_m = tm;
  p.tiles_n = (a->N + bn - 1) / bn;
  p.num_kb = num_kb;
  p.splits = splits;
  p.kb_per_split = (num_kb + splits - 1) / splits;
  if ((long long)(splits - 1) * p.kb_per_split >= num_kb) {  // keep every split non-empty
    splits = (num_kb + p.kb_per_split - 1) / p.kb_per_split;
    p.splits = splits;
  }
  p.ws = static_cast<float*>(a->ws);
  p.counters = a->counters;
  if (ar) {
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    if (p.splits != 1 || tiles > ar->max_tiles || tiles * bn * kBM > ar->partial_elems) return kErrTooLarge;
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
    p.ar.mode = ar->mode == 1 ? 1 : 0;
    p.ar.rows_per_rank = a->M / ar->world;
  }
  if (ag) {
    p.ag.world = ag->world;
    p.ag.rank = ag->rank;
    p.ag.tiles_per_rank = (int)(ag->rows_per_rank / kBM);
    p.ag.ready = static_cast<const uint32_t*>(ag->ready);
    p.ag.epoch = static_cast<const uint32_t*>(ag->epoch);
    p.row_epi = (!p.out_f32 && p.vec_ok && !(p.bias && p.bias_f32)) ? 1 : 0;
    TmapSet peers;
    for (int r = 0; r < kMaxRanks; ++r) {
      const int src = r < ag->world ? r : ag->rank;
      if (!al16(ag->a_peer[src])) return kErrBadShape;
      const int rc_a = encode_tmap_2d_bf16(&peers.m[r], ag->a_peer[src], (uint64_t)a->K, (uint64_t)ag->rows_per_rank,
                                           (uint64_t)a->lda * 2, 64, kBM);
      if (rc_a) return rc_a;
    }
    CUtensorMap tmBg;
    const int rc_b = encode_tmap_2d_bf16(&tmBg, a->B, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->ldb * 2, 64, (uint32_t)bn);
    if (rc_b) return rc_b;
    return bn == 256 ? launch_tc_ag<256, 4>(peers, tmBg, p, stream) : launch_tc_ag<128, 6>(peers, tmBg, p, stream);
  }

  CUtensorMap tmA, tmB;
  int rc;
  if (a->trans_a) rc = encode_tmap_2d_bf16(&tmA, a->A, (uint64_t)a->M, (uint64_t)a->K, (uint64_t)a->lda * 2, 64, 64);
  else            rc = encode_tmap_2d_bf16(&tmA, a->A, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->lda * 2, 64, kBM);
  if (rc) return rc;
  if (a->trans_b) rc = encode_tmap_2d_bf16(&tmB, a->B, (uint64_t)a->K, (uint64_t)a->N, (uint64_t)a->ldb * 2, 64,
                                           (uint32_t)(pair ? bn / 2 : bn));
  else            rc = encode_tmap_2d_bf16(&tmB, a->B, (uint64_t)a->N, (uint64_t)a->K, (uint64_t)a->ldb * 2, 64, 64);
  if (rc) return rc;

  // bf16 outputs take the row-per-thread register epilogue (DPTB_GEMM_STAGED_EPILOGUE=1 keeps the staged one, for
  // comparisons); 32-byte accesses when every per-element buffer allows them.
  static const bool staged_only = [] {
    const char* e = getenv("DPTB_GEMM_STAGED_EPILOGUE");
    return e && e[0] == '1';
  }();
  p.row_epi = (!ar && !staged_only && !p.out_f32 && p.vec_ok && !(p.bias && p.bias_f32)) ? 1 : 0;
  if (p.row_epi) {
    auto wide_ok = [](const void* q, long long ld) { return (reinterpret_cast<uintptr_t>(q) & 31) == 0 && ld % 16 == 0; };
    if (wide_ok(p.C, p.ldc) && (!p.residual || wide_ok(p.residual, p.ldr)) &&
        (!p.aux_out || wide_ok(p.aux_out, p.ld_aux_out)) && (!p.aux_in || wide_ok(p.aux_in, p.ld_aux_in)))
      p.row_epi = 2;
  }

  // CTA pairs with a bf16 output take the tile-store epilogue when every per-element buffer can be described by a
  // tensor map (16-byte aligned, row strides multiples of 16 bytes: vec_ok), at most one per-element input is read
  // and a pre-activation copy is not combined with an input (the two staging blocks of a warp cover either case).
  EpiMaps em;
  if (pair && p.splits == 1) {
    const int inputs = epi_inputs;
    {
      const void* in_ptr = p.act >= 11 ? (const void*)p.aux_in : (p.residual ? (const void*)p.residual : p.C);
      const long long in_ld = p.act >= 11 ? p.ld_aux_in : (p.residual ? p.ldr : p.ldc);
      int e = encode_tmap_2d_bf16(&em.c, p.C, (uint64_t)a->N, (uint64_t)a->M, (uint64_t)p.ldc * 2, 64, 32);
      if (!e) e = p.aux_out ? encode_tmap_2d_bf16(&em.aux, p.aux_out, (uint64_t)a->N, (uint64_t)a->M,
                                                  (uint64_t)p.ld_aux_out * 2, 64, 32)
                            : (em.aux = em.c, 0);
      if (!e) e = inputs ? encode_tmap_2d_bf16(&em.in, in_ptr, (uint64_t)a->N, (uint64_t)a->M, (uint64_t)in_ld * 2, 64, 32)
                         : (em.in = em.c, 0);
      if (e) return e;
      p.row_epi = 3;
    }
  }
  if (p.row_epi != 3) em.c = em.aux = em.in = tmA;   // unused by the kernel, but kernel parameters must be initialised

  const bool amn = a->trans_a != 0, bmn = a->trans_b == 0;
#define DPTB_LAUNCH(AMN, BMN)                                                                                         \
  (pair ? (bn == 256 ? launch_tc_pair<AMN, BMN, 256, kPairStages256>(tmA, tmB, em, p, stream)                          \
                     : launch_tc_pair<AMN, BMN, 128, kPairStages128>(tmA, tmB, em, p, stream))                         \
        : (bn == 256 ? launch_tc<AMN, BMN, 256, 4>(tmA, tmB, p, stream) : launch_tc<AMN, BMN, 128, 6>(tmA, tmB, p, stream)))
  if (!amn && !bmn) return DPTB_LAUNCH(false, false);
  if (!amn && bmn) return DPTB_LAUNCH(false, true);
  if (amn && !bmn) return DPTB_LAUNCH(true, false);
  return DPTB_LAUNCH(true, true);
#undef DPTB_LAUNCH
}

extern "C" int dptb_gemm(const DptbGemmArgs* a, void* stream_v) { return gemm_impl(a, nullptr, nullptr, stream_v); }
// Row-parallel Linear of a tensor-parallel group in ONE kernel: tcgen05 GEMM of this rank's K-slice, then the sum over
// ranks (+ bias, + residual) through NVLink peer memory, delivered to every rank's `out`.  Every rank must call it with
// the same shapes; C of the argument block is ignored (the result goes to ar->out_peer / ar->mc_out with row stride ldc).
extern "C" int dptb_gemm_allreduce(const DptbGemmArgs* a, const DptbTpArArgs* ar, void* stream_v) {
  if (!ar) return kErrBadShape;
  return gemm_impl(a, ar, nullptr, stream_v);
}
// Column-parallel Linear on a row-sharded input in ONE kernel: row tile i of A is read by TMA straight from the
// symmetric buffer of the rank that owns those rows, once that rank's dptb_tp_signal has published the shard; the
// output [M, N] (this rank's slice of the features, all rows) is local.  A of the argument block is ignored.
extern "C" int dptb_allgather_gemm(const DptbGemmArgs* a, const DptbTpAgArgs* ag, void* stream_v) {
  if (!ag) return kErrBadShape;
  return gemm_impl(a, nullptr, ag, stream_v);
}

// Publishes "this rank's shard is complete" to every peer: flag word [rank] of each peer's `ready` array and the local
// launch counter both become *epoch + 1.  Runs after the kernel that wrote the shard, in stream order.
struct DptbTpSignalArgs {
  int world, rank;
  void* ready_peer[kMaxRanks];   // every rank's flag array [kMaxRanks]
  void* epoch;                   // local launch counter
};
namespace dptb {
struct SignalParams {
  int world, rank;
  uint32_t* ready_peer[kMaxRanks];
  uint32_t* epoch;
};
__global__ void tp_shard_signal_kernel(const SignalParams s) {
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(s.epoch) + 1u;
  __threadfence_system();   // the shard written by earlier kernels of this stream is visible system-wide first
  if ((int)threadIdx.x < s.world) st_release_sys(s.ready_peer[threadIdx.x] + s.rank, e);
  __syncwarp();
  if (threadIdx.x == 0) *s.epoch = e;
}
}  // namespace dptb
extern "C" int dptb_tp_signal(const DptbTpSignalArgs* a, void* stream_v) {
  if (!a || a->world < 1 || a->world > kMaxRanks) return kErrBadShape;
  SignalParams s;
  s.world = a->world;
  s.rank = a->rank;
  for (int r = 0; r < kMaxRanks; ++r) s.ready_peer[r] = static_cast<uint32_t*>(a->ready_peer[r]);
  s.epoch = static_cast<uint32_t*>(a->epoch);
  tp_shard_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_v)>>>(s);
  return counted(1, (int)cudaGetLastError());
}

// Stream-ordered wait for the peers' shards: returns once every other rank's "shard ready" flag in THIS rank's flag
// array has reached this rank's own publication count (so it runs after this rank's dptb_tp_signal).  Each wait is
// bounded; one that runs out is recorded in the status word and the kernel returns all the same.  What follows it on
// the stream (copies of the peers' shards into local memory) then sees complete shards.
namespace dptb {
__global__ void tp_wait_ready_kernel(const uint32_t* ready, const uint32_t* epoch, int world, int rank) {
  const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(epoch);
  const int src = threadIdx.x;
  if (src < world && src != rank) wait_flag_ge(ready + src, e);
}
}  // namespace dptb
// One device-to-device copy on the stream by the copy engines (no SM is taken from the GEMM that runs beside it);
// either pointer may be peer-mapped memory.
extern "C" int dptb_copy_async(void* dst, const void* src, long long nbytes, void* stream_v) {
  if (nbytes <= 0) return 0;
  if (!dst || !src) return kErrBadShape;
  return (int)cudaMemcpyAsync(dst, src, (size_t)nbytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream_v));
}
extern "C" int dptb_tp_wait_ready(const void* ready, const void* epoch, int world, int rank, void* stream_v) {
  if (!ready || !epoch || world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return kErrBadShape;
  tp_wait_ready_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_v)>>>(
      static_cast<const uint32_t*>(ready), static_cast<const uint32_t*>(epoch), world, rank);
  return counted(1, (int)cudaGetLastError());
}

// Status word access ------------------------------------------------------------------------------
// Folds the blocks of all translation units: the first non-zero code (with its detail) and the total number of
// waits that ran out.
extern "C" int dptb_status_read(int* out4) {
  out4[0] = out4[1] = out4[2] = out4[3] = 0;
  for (int i = 0; i < g_num_status_blocks; ++i) {
    int b[4] = {0, 0, 0, 0};
    const int rc = g_status_blocks[i](b, 0);
    if (rc) return rc;
    if (out4[0] == 0 && b[0] != 0) { out4[0] = b[0]; out4[1] = b[1]; }
    out4[2] += b[2];
  }
  return 0;
}
extern "C" int dptb_status_clear() {
  for (int i = 0; i < g_num_status_blocks; ++i) {
    const int rc = g_status_blocks[i](nullptr, 1);
    if (rc) return rc;
  }
  return 0;
}

// Role timers (see DPTB_GEMM_PROFILE): copies [256][12] counters out and zeroes them; -5 when not compiled in.
extern "C" int dptb_gemm_profile_read(unsigned long long* out) {
#ifdef DPTB_GEMM_PROFILE
  int rc = (int)cudaMemcpyFromSymbol(out, g_gemm_prof, sizeof(unsigned long long) * 256 * kProfSlots);
  if (rc) return rc;
  static unsigned long long zeros[256 * kProfSlots];
  return (int)cudaMemcpyToSymbol(g_gemm_prof, zeros, sizeof(zeros));
#else
  (void)out;
  return kErrUnsupported;
#endif
}

extern "C" long long dptb_launch_count() { return launch_counter(); }
extern "C" void dptb_launch_count_reset() { launch_counter() = 0; }
