// Expert-parallel mixture-of-experts: routing, and the all-to-all dispatch / return of token rows done by the kernels
// themselves with peer stores over NVLink (no collective library on the data path).
//
// The reference keeps all experts on one device; its sparse path gathers routed rows, runs the expert and scatter-adds
// the weighted result (reference: lib/core/nn/moe.dart:479-522, lib/core/tensor/scatter.dart:23-84).  Here experts are
// sharded over the ranks of a group (`El` local experts per rank, `E = El * world` in all).  Every (source rank, expert)
// pair owns a fixed quota of `C` rows, so all buffers are static:
//
//   recv[El][world][C][D]   on the expert's rank: rows that arrived for local expert le from source rank s
//   ret [E][C][D]           on the source rank: expert outputs for the rows this rank sent, by (expert, slot)
//
//   moe_route_kernel     softmax over the router logits, top-k, optional renormalisation          (per token)
//   moe_slot_kernel      slot of every (token, choice) inside its expert's quota, in token order; -1 = dropped
//   moe_dispatch_kernel  row t -> recv[le][me][slot] on the owner of expert e (16-byte peer stores, optional per-row
//                        scale), then per-expert counts and a flag to every peer, then a bounded wait for every peer's
//                        flag: when the kernel completes on a rank, all rows sent TO that rank have landed
//   moe_zero_tail_kernel rows [count, C) of every (local expert, source) quota := 0, so the dense expert GEMMs over
//                        the whole buffer add nothing for unused slots (forward outputs and weight gradients)
//   moe_return_kernel    expert-side rows of source s -> ret[e][0:count] on rank s, same flag protocol
//   moe_combine_kernel   y[t] = sum_j w[t][j] * ret[e_j][slot_j]        (weights optional: 1)
//   moe_combine_dot      dw[t][j] = <dy[t], ret[e_j][slot_j]>           (gradient of the routing weights)
// The backward pass reuses them: dy rows scaled by w are dispatched, the expert backward runs on them, the input
// gradients are returned and combined with unit weights.  Epoch words live on the device (CUDA-graph replay).
#include <cuda_bf16.h>

#include "common/host.h"
#include "common/peer.cuh"
#include "common/reduce.cuh"

namespace dptb {

constexpr int kMaxExperts = 64;
constexpr int kMaxTopK = 8;

// ---------------------------------------------------------------------------------------------- routing
// logits [T, ld] fp32 or bf16 -> probs [T, E] fp32, idx [T, k] int32, w [T, k] fp32.
//   gate 0: probs = softmax(logits); gate 1: probs = sigmoid(logits) (reference: lib/core/nn/moe.dart:379-472).
//   The choice is made on probs + bias (aux-loss-free balancing bias, may be null; the weights stay unbiased).
//   groups > 1: the experts form `groups` equal groups; a group's score is its best biased score (softmax gate) or the
//   sum of its two best (sigmoid gate); only experts of the `top_groups` best groups can be chosen.
template <typename TL>
__global__ void __launch_bounds__(256)
moe_route_kernel(const TL* __restrict__ logits, long long ld, float* __restrict__ probs, int* __restrict__ idx,
                 float* __restrict__ w, int T, int E, int k, int renorm, float route_scale, int gate,
                 const float* __restrict__ bias, int groups, int top_groups) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float p[kMaxExperts];
  if (gate == 0) {
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) {
      p[e] = to_f32(logits[(long long)t * ld + e]);
      mx = fmaxf(mx, p[e]);
    }
    float sum = 0.0f;
    for (int e = 0; e < E; ++e) {
      p[e] = __expf(p[e] - mx);
      sum += p[e];
    }
    const float inv = 1.0f / sum;
    for (int e = 0; e < E; ++e) p[e] *= inv;
  } else {
    for (int e = 0; e < E; ++e) p[e] = 1.0f / (1.0f + __expf(-to_f32(logits[(long long)t * ld + e])));
  }
  for (int e = 0; e < E; ++e) probs[(long long)t * E + e] = p[e];
  // scores the choice is made on; experts of groups that are not kept drop to -inf
  float sel[kMaxExperts];
  for (int e = 0; e < E; ++e) sel[e] = p[e] + (bias ? bias[e] : 0.0f);
  if (groups > 1) {
    const int per = E / groups;
    float gs[kMaxExperts];
    for (int g = 0; g < groups; ++g) {
      float b1 = -INFINITY, b2 = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float v = sel[e];
        if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
      }
      gs[g] = (gate == 1 && per >= 2) ? b1 + b2 : b1;
    }
    unsigned long long keep = 0ull;
    for (int j = 0; j < top_groups; ++j) {
      int best = -1;
      float bv = -INFINITY;
      for (int g = 0; g < groups; ++g)
        if (!((keep >> g) & 1ull) && (best < 0 || gs[g] > bv)) { bv = gs[g]; best = g; }
      keep |= 1ull << best;
    }
    for (int e = 0; e < E; ++e)
      if (!((keep >> (e / per)) & 1ull)) sel[e] = -INFINITY;
  }
  float wsum = 0.0f;
  unsigned long long taken = 0ull;
  for (int j = 0; j < k; ++j) {
    int best = -1;
    float bv = -INFINITY;
    for (int e = 0; e < E; ++e)
      if (!((taken >> e) & 1ull) && (best < 0 || sel[e] > bv)) {      // ties resolve to the lowest expert index
        bv = sel[e];
        best = e;
      }
    taken |= 1ull << best;
    idx[(long long)t * k + j] = best;
    w[(long long)t * k + j] = p[best];
    wsum += p[best];
  }
  const float s = (renorm ? 1.0f / (wsum + 1e-9f) : 1.0f) * route_scale;
  for (int j = 0; j < k; ++j) w[(long long)t * k + j] *= s;
}

// One CTA per expert walks all (token, choice) pairs in order: slot = number of earlier pairs routed to this expert.
__global__ void __launch_bounds__(1024)
moe_slot_kernel(const int* __restrict__ idx, int* __restrict__ slot, int* __restrict__ count, int n_pairs, int C) {
  __shared__ int warp_tot[32];
  __shared__ int base;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) base = 0;
  __syncthreads();
  for (int i0 = 0; i0 < n_pairs; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    const int hit = (i < n_pairs && idx[i] == e) ? 1 : 0;
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    const int before = __popc(ballot & ((1u << lane) - 1));
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int off = base;
    for (int wv = 0; wv < warp; ++wv) off += warp_tot[wv];
    if (hit) {
      const int s = off + before;
      slot[i] = s < C ? s : -1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int wv = 0; wv < (int)(blockDim.x >> 5); ++wv) tot += warp_tot[wv];
      base += tot;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) count[e] = base < C ? base : C;
}

// ---------------------------------------------------------------------------------------------- dispatch / return
struct EpArgs {
  int world, rank, El, C, D, E;
  __nv_bfloat16* recv_peer[kMaxRanks];   // recv buffer of every rank  [El][world][C][D]
  __nv_bfloat16* ret_peer[kMaxRanks];    // ret buffer of every rank   [E][C][D]
  int* counts_peer[kMaxRanks];           // [El][world] rows that source s sent to local expert le (on the expert rank)
  uint32_t* flags_peer[kMaxRanks];       // [2][kMaxRanks]: dispatch-done[src], return-done[src]
  uint32_t* epoch;                       // local [2]: dispatch launches, return launches
  unsigned int* exit_counter;            // local [2]
};

__device__ __forceinline__ void ep_end_barrier(const EpArgs& a, int which, uint32_t e) {
  // Last CTA of this rank: everything this rank had to send is written; tell every peer, wait for every peer.
  __threadfence_system();
  if (atomicAdd(a.exit_counter + which, 1u) == gridDim.x - 1) {
    a.exit_counter[which] = 0;
    __threadfence_system();
    for (int r = 0; r < a.world; ++r) st_release_sys(a.flags_peer[r] + which * kMaxRanks + a.rank, e);
    for (int r = 0; r < a.world; ++r)
      if (!wait_flag_ge(a.flags_peer[a.rank] + which * kMaxRanks + r, e)) break;
    a.epoch[which] = e;
  }
}

// One warp per (token, choice) pair.  x [T, ldx]; idx / slot [T * k]; scale [T * k] or null.
__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const EpArgs a, const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ idx,
                    const int* __restrict__ slot, const float* __restrict__ scale, const int* __restrict__ count,
                    int n_pairs, int k) {
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(a.epoch) + 1u;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = a.D / 8;
  for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < n_pairs; i += gridDim.x * wpb) {
    const int s = slot[i];
    if (s < 0) continue;
    const int ex = idx[i];
    const int owner = ex / a.El, le = ex % a.El;
    const __nv_bfloat16* src = x + (long long)(i / k) * ldx;
    __nv_bfloat16* dst = a.recv_peer[owner] + (((long long)le * a.world + a.rank) * a.C + s) * a.D;
    const float sc = scale ? scale[i] : 1.0f;
    for (int v = lane; v < nvec; v += 32) {
      uint4 u = *reinterpret_cast<const uint4*>(src + v * 8);
      if (scale) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(h[q]);
          h[q] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
      }
      st_cg_v4(dst + v * 8, u);
    }
  }
  // counts: this rank's row count for every expert goes to the expert's owner
  if (blockIdx.x == 0 && threadIdx.x < a.E) {
    const int ex = threadIdx.x;
    a.counts_peer[ex / a.El][(ex % a.El) * a.world + a.rank] = count[ex];
  }
  __syncthreads();
  if (threadIdx.x == 0) ep_end_barrier(a, 0, e);
}

// rows [El][world][C][D] (this rank's expert outputs) -> ret[e][slot] on every source rank.
__global__ void __launch_bounds__(256)
moe_return_kernel(const EpArgs a, const __nv_bfloat16* __restrict__ rows, const int* __restrict__ counts_local) {
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(a.epoch + 1) + 1u;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = a.D / 8;
  const long long total = (long long)a.El * a.world * a.C;
  for (long long i = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); i < total; i += (long long)gridDim.x * wpb) {
    const int s = (int)(i % a.C);
    const int src_rank = (int)((i / a.C) % a.world);
    const int le = (int)(i / ((long long)a.C * a.world));
    if (s >= counts_local[le * a.world + src_rank]) continue;
    const __nv_bfloat16* src = rows + i * a.D;
    __nv_bfloat16* dst = a.ret_peer[src_rank] + (((long long)(a.rank * a.El + le)) * a.C + s) * a.D;
    for (int v = lane; v < nvec; v += 32) st_cg_v4(dst + v * 8, *reinterpret_cast<const uint4*>(src + v * 8));
  }
  __syncthreads();
  if (threadIdx.x == 0) ep_end_barrier(a, 1, e);
}

// rows [El][world][C][D]: zero the unused tail of every quota.
__global__ void __launch_bounds__(256)
moe_zero_tail_kernel(__nv_bfloat16* __restrict__ rows, const int* __restrict__ counts_local, int El, int world, int C,
                     int D) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = D / 8;
  const long long total = (long long)El * world * C;
  for (long long i = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); i < total; i += (long long)gridDim.x * wpb) {
    const int s = (int)(i % C);
    const int q = (int)(i / C);                  // le * world + src
    if (s < counts_local[q]) continue;
    uint4* dst = reinterpret_cast<uint4*>(rows + i * D);
    for (int v = lane; v < nvec; v += 32) dst[v] = make_uint4(0, 0, 0, 0);
  }
}

// y[t] = sum_j w[t][j] * ret[idx][slot]; one warp per token.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ ret, const int* __restrict__ idx, const int* __restrict__ slot,
                   const float* __restrict__ w, __nv_bfloat16* __restrict__ y, long long ldy, int T, int k, int C, int D) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = D / 8;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int j = 0; j < k; ++j) {
        const int s = slot[t * k + j];
        if (s < 0) continue;
        const float wj = w ? w[t * k + j] : 1.0f;
        float f[8];
        Vec8<__nv_bfloat16>::load(ret + (((long long)idx[t * k + j]) * C + s) * D + v * 8, f);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = fmaf(wj, f[q], acc[q]);
      }
      Vec8<__nv_bfloat16>::store(y + (long long)t * ldy + v * 8, acc);
    }
  }
}

// dw[t][j] = <dy[t], ret[idx][slot]>; one warp per (token, choice).
__global__ void __launch_bounds__(256)
moe_combine_dot_kernel(const __nv_bfloat16* __restrict__ ret, const int* __restrict__ idx,
                       const int* __restrict__ slot, const __nv_bfloat16* __restrict__ dy, long long lddy,
                       float* __restrict__ dw, int n_pairs, int k, int C, int D) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = D / 8;
  for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < n_pairs; i += gridDim.x * wpb) {
    const int s = slot[i];
    float acc = 0.0f;
    if (s >= 0) {
      const __nv_bfloat16* r = ret + (((long long)idx[i]) * C + s) * D;
      const __nv_bfloat16* g = dy + (long long)(i / k) * lddy;
      for (int v = lane; v < nvec; v += 32) {
        float a8[8], b8[8];
        Vec8<__nv_bfloat16>::load(r + v * 8, a8);
        Vec8<__nv_bfloat16>::load(g + v * 8, b8);
#pragma unroll
        for (int q = 0; q < 8; ++q) acc = fmaf(a8[q], b8[q], acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dw[i] = acc;
  }
}

}  // namespace dptb

using namespace dptb;

struct DptbEpArgs {
  int world, rank, El, C, D, E;
  void* recv_peer[kMaxRanks];
  void* ret_peer[kMaxRanks];
  void* counts_peer[kMaxRanks];
  void* flags_peer[kMaxRanks];
  void* epoch;
  void* exit_counter;
};

static int fill_ep(const DptbEpArgs* h, EpArgs* a) {
  if (h->world < 1 || h->world > kMaxRanks || h->rank < 0 || h->rank >= h->world) return kErrBadShape;
  if (h->El < 1 || h->E != h->El * h->world || h->E > kMaxExperts || h->C < 1 || h->D < 8 || (h->D % 8)) return kErrBadShape;
  a->world = h->world; a->rank = h->rank; a->El = h->El; a->C = h->C; a->D = h->D; a->E = h->E;
  for (int r = 0; r < kMaxRanks; ++r) {
    a->recv_peer[r] = static_cast<__nv_bfloat16*>(h->recv_peer[r]);
    a->ret_peer[r] = static_cast<__nv_bfloat16*>(h->ret_peer[r]);
    a->counts_peer[r] = static_cast<int*>(h->counts_peer[r]);
    a->flags_peer[r] = static_cast<uint32_t*>(h->flags_peer[r]);
  }
  a->epoch = static_cast<uint32_t*>(h->epoch);
  a->exit_counter = static_cast<unsigned int*>(h->exit_counter);
  return 0;
}
static inline int ep_grid(long long warps) {
  const long long want = (warps + 7) / 8;
  const long long cap = (long long)sm_count() * 8;
  return (int)(want < 1 ? 1 : (want > cap ? cap : want));
}

extern "C" int dptb_moe_route(const void* logits, long long ld, int logits_f32, float* probs, int* idx, float* w, int T,
                              int E, int k, int renorm, float route_scale, int gate, const float* bias, int groups,
                              int top_groups, void* stream) {
  if (T <= 0) return 0;
  if (E < 1 || E > kMaxExperts || k < 1 || k > kMaxTopK || k > E || (gate != 0 && gate != 1)) return kErrBadShape;
  if (groups < 1) groups = 1;
  if (groups > 1 && (E % groups || top_groups < 1 || top_groups > groups || k > top_groups * (E / groups))) return kErrBadShape;
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = (T + 255) / 256;
  if (logits_f32) moe_route_kernel<float><<<grid, 256, 0, st>>>((const float*)logits, ld, probs, idx, w, T, E, k, renorm, route_scale, gate, bias, groups, top_groups);
  else moe_route_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)logits, ld, probs, idx, w, T, E, k, renorm, route_scale, gate, bias, groups, top_groups);
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_moe_slots(const int* idx, int* slot, int* count, int n_pairs, int E, int C, void* stream) {
  if (n_pairs <= 0) return 0;
  moe_slot_kernel<<<E, 1024, 0, static_cast<cudaStream_t>(stream)>>>(idx, slot, count, n_pairs, C);
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_moe_dispatch(const DptbEpArgs* h, const void* x, long long ldx, const int* idx, const int* slot,
                                 const float* scale, const int* count, int T, int k, void* stream) {
  EpArgs a;
  if (int rc = fill_ep(h, &a)) return rc;
  if (T <= 0 || (ldx % 8) || (reinterpret_cast<uintptr_t>(x) & 15)) return kErrBadShape;
  const int n_pairs = T * k;
  moe_dispatch_kernel<<<ep_grid(n_pairs), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      a, static_cast<const __nv_bfloat16*>(x), ldx, idx, slot, scale, count, n_pairs, k);
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_moe_zero_tail(void* rows, const int* counts_local, int El, int world, int C, int D, void* stream) {
  if ((D % 8) || (reinterpret_cast<uintptr_t>(rows) & 15)) return kErrBadShape;
  moe_zero_tail_kernel<<<ep_grid((long long)El * world * C), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(rows), counts_local, El, world, C, D);
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_moe_return(const DptbEpArgs* h, const void* rows, const int* counts_local, void* stream) {
  EpArgs a;
  if (int rc = fill_ep(h, &a)) return rc;
  if (reinterpret_cast<uintptr_t>(rows) & 15) return kErrBadShape;
  moe_return_kernel<<<ep_grid((long long)a.El * a.world * a.C), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      a, static_cast<const __nv_bfloat16*>(rows), counts_local);
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_moe_combine(const void* ret, const int* idx, const int* slot, const float* w, void* y, long long ldy,
                                int T, int k, int C, int D, void* stream) {
  if (T <= 0) return 0;
  if ((D % 8) || (ldy % 8)) return kErrBadShape;
  moe_combine_kernel<<<ep_grid(T), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(ret), idx, slot, w, static_cast<__nv_bfloat16*>(y), ldy, T, k, C, D);
  return counted(1, (int)cudaGetLastError());
}
extern "C" int dptb_moe_combine_dot(const void* ret, const int* idx, const int* slot, const void* dy, long long lddy,
                                    float* dw, int T, int k, int C, int D, void* stream) {
  if (T <= 0) return 0;
  if ((D % 8) || (lddy % 8)) return kErrBadShape;
  moe_combine_dot_kernel<<<ep_grid((long long)T * k), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(ret), idx, slot, static_cast<const __nv_bfloat16*>(dy), lddy, dw, T * k, k, C, D);
  return counted(1, (int)cudaGetLastError());
}
