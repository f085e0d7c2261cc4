// Small tensor-parallel collectives that would otherwise cost a library call per decode step.
//
// tp_argmax_kernel: greedy next token over a vocabulary-sharded logits matrix.  Every rank holds logits[B, Vl] for its
// slice of the vocabulary.  CTA b finds the local (max, argmax) of row b, writes the pair (value, global index) into
// slot [b][rank] of EVERY rank's symmetric exchange buffer with plain peer stores, raises flag[b][rank] on every peer,
// waits (bounded) for the other ranks' flags of row b and picks the winner (largest value, lowest index on ties), so
// all ranks end up with the same token ids without any round trip to the host.  Epochs count launches (the word lives
// on the device), so a captured CUDA graph can replay the kernel.
#include <cuda_bf16.h>

#include "common/host.h"
#include "common/peer.cuh"
#include "common/reduce.cuh"

namespace dptb {

struct TpArgmaxArgs {
  const __nv_bfloat16* logits;     // [B, ld]
  long long ld;
  int B, Vl, vocab_offset, rank, world;
  float* xchg_peer[kMaxRanks];     // every rank's exchange buffer: [2][B][kMaxRanks][2] floats (value, index bits);
                                   // the leading index is the launch parity, so a fast rank's next launch cannot
                                   // overwrite a pair that a slow rank has not read yet
  uint32_t* flags_peer[kMaxRanks]; // every rank's flags: [B][kMaxRanks]
  long long* tokens;               // [B] out (local)
  uint32_t* epoch;                 // local launch counter
  unsigned int* exit_counter;      // local
  int* pos_ptr;                    // optional: incremented by `pos_inc` by the last CTA (decode position)
  int pos_inc;
};

__global__ void __launch_bounds__(256)
tp_argmax_kernel(const TpArgmaxArgs a) {
  __shared__ float s_val[256];
  __shared__ int s_idx[256];
  const int b = blockIdx.x;
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(a.epoch) + 1u;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const __nv_bfloat16* row = a.logits + (long long)b * a.ld;
  int i0 = 0;
  if ((a.ld % 8) == 0 && (reinterpret_cast<uintptr_t>(a.logits) & 15) == 0) {
    // 16-byte loads, four in flight per thread
    const int nv = a.Vl / 8;
    for (int v0 = threadIdx.x; v0 < nv; v0 += 4 * blockDim.x) {
      uint4 u[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int vi = v0 + k * blockDim.x;
        u[k] = vi < nv ? *reinterpret_cast<const uint4*>(row + (long long)vi * 8) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int vi = v0 + k * blockDim.x;
        if (vi >= nv) continue;
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u[k]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float v = __bfloat162float(e[j]);
          const int i = vi * 8 + j;
          if (v > best || (v == best && i < best_i)) {
            best = v;
            best_i = i;
          }
        }
      }
    }
    i0 = nv * 8;
  }
  for (int i = i0 + threadIdx.x; i < a.Vl; i += blockDim.x) {
    const float v = __bfloat162float(row[i]);
    if (v > best || (v == best && i < best_i)) {
      best = v;
      best_i = i;
    }
  }
  s_val[threadIdx.x] = best;
  s_idx[threadIdx.x] = best_i;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if (threadIdx.x < off) {
      const float v = s_val[threadIdx.x + off];
      const int i = s_idx[threadIdx.x + off];
      if (v > s_val[threadIdx.x] || (v == s_val[threadIdx.x] && i < s_idx[threadIdx.x])) {
        s_val[threadIdx.x] = v;
        s_idx[threadIdx.x] = i;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x < a.world) {
    const int r = threadIdx.x;
    float* slot = a.xchg_peer[r] + (((long long)(e & 1) * a.B + b) * kMaxRanks + a.rank) * 2;
    slot[0] = s_val[0];
    slot[1] = __int_as_float(s_idx[0] + a.vocab_offset);
    __threadfence_system();
    st_release_sys(a.flags_peer[r] + (long long)b * kMaxRanks + a.rank, e);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float win = -INFINITY;
    int win_i = 0x7fffffff;
    bool ok = true;
    for (int r = 0; r < a.world && ok; ++r) {
      ok = wait_flag_ge(a.flags_peer[a.rank] + (long long)b * kMaxRanks + r, e);
      if (!ok) break;
      const volatile float* slot = a.xchg_peer[a.rank] + (((long long)(e & 1) * a.B + b) * kMaxRanks + r) * 2;
      const float v = slot[0];
      const int i = __float_as_int(slot[1]);
      if (v > win || (v == win && i < win_i)) {
        win = v;
        win_i = i;
      }
    }
    a.tokens[b] = ok ? (long long)win_i : -1;
    __threadfence();
    if (atomicAdd(a.exit_counter, 1u) == gridDim.x - 1) {
      *a.exit_counter = 0;
      *a.epoch = e;
      if (a.pos_ptr) *a.pos_ptr += a.pos_inc;
    }
  }
}

}  // namespace dptb

using namespace dptb;

struct DptbTpArgmaxArgs {
  const void* logits;
  long long ld;
  int B, Vl, vocab_offset, rank, world;
  void* xchg_peer[kMaxRanks];
  void* flags_peer[kMaxRanks];
  void* tokens;
  void* epoch;
  void* exit_counter;
  void* pos_ptr;
  int pos_inc;
};

extern "C" int dptb_tp_argmax(const DptbTpArgmaxArgs* h, void* stream) {
  if (h->B <= 0) return 0;
  if (h->world < 1 || h->world > kMaxRanks || h->rank < 0 || h->rank >= h->world || h->Vl <= 0) return kErrBadShape;
  TpArgmaxArgs a;
  a.logits = static_cast<const __nv_bfloat16*>(h->logits);
  a.ld = h->ld; a.B = h->B; a.Vl = h->Vl; a.vocab_offset = h->vocab_offset; a.rank = h->rank; a.world = h->world;
  for (int r = 0; r < kMaxRanks; ++r) {
    a.xchg_peer[r] = static_cast<float*>(h->xchg_peer[r]);
    a.flags_peer[r] = static_cast<uint32_t*>(h->flags_peer[r]);
  }
  a.tokens = static_cast<long long*>(h->tokens);
  a.epoch = static_cast<uint32_t*>(h->epoch);
  a.exit_counter = static_cast<unsigned int*>(h->exit_counter);
  a.pos_ptr = static_cast<int*>(h->pos_ptr);
  a.pos_inc = h->pos_inc;
  tp_argmax_kernel<<<h->B, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return counted(1, (int)cudaGetLastError());
}
