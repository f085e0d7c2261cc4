// Data-parallel gradient all-reduce over NVLink / NVSwitch peer memory, fused with the sum-of-squares partials that
// gradient clipping needs.  No NCCL call: the kernel itself issues multimem (in-switch reduction) or plain peer
// loads / stores and synchronises ranks through flag words in a symmetric signal buffer.
//
// It replaces the reference's only multi-replica mechanism, averaging whole checkpoints on the CPU every K local steps
// (reference: lib/core/coop/param_avg.dart:20-123), with synchronous intra-node data parallelism.
//
// Layout.  Every rank holds the same flat bf16 gradient buffer in symmetric memory; `bases[r]` is rank r's copy mapped
// into this process, `mc_base` the multicast address of all copies (0 when the fabric has none).  A launch handles one
// bucket [start, start + n).  Rank r owns the r-th slice of the bucket: it reads that slice from every rank, adds in
// fp32 in rank order, scales by 1 / world, writes the average back into every rank's copy, and accumulates the sum of
// squares of what it wrote.
//
// Protocol per bucket b (epoch e = launches of this bucket so far, kept in device memory so CUDA graphs can replay):
//   ready[b][src] = e   written into every peer's signal buffer at kernel start (stream order puts it after the
//                       backward kernels that produced the bucket)
//   wait until ready[b][*] >= e locally (bounded), then reduce the owned slice
//   last CTA of the grid: fold the per-CTA sums in CTA order, publish sumsq[b][rank] and done[b][rank] = e to every peer
// dp_finalize waits (bounded) for done[*][*] >= e, adds sumsq[*][*] in fixed order and writes the clip control block
// {norm, scale, finite, sumsq}; the optimizer kernel that follows therefore sees fully reduced gradients.
// Every wait is bounded (`wait_ns`, a launch argument: it is the largest skew between ranks a step tolerates).  A
// wait that runs out records kWaitFlagTimeout in the status word, and the rank publishes NaN as its sum of squares, so
// every rank's control block reads "not finite" and an optimizer told to skip such steps leaves the weights alone.
#include <cuda_bf16.h>

#include "common/host.h"
#include "common/peer.cuh"
#include "common/ptx.cuh"
#include "common/reduce.cuh"

namespace dptb {

constexpr int kDpThreads = 512;

struct DpArgs {
  __nv_bfloat16* bases[kMaxRanks];   // flat gradient buffer of every rank
  uint32_t* pads[kMaxRanks];         // signal buffer of every rank
  __nv_bfloat16* mc_base;            // multicast address of the gradient buffers, or null
  int rank, world;
  int bucket, num_buckets;
  long long start, n;                // element range of this bucket (multiples of 8)
  float* cta_partial;                // local scratch [gridDim.x]
  unsigned int* cta_counter;         // local, zero between launches
  unsigned int* epochs;              // local [num_buckets]
  unsigned long long wait_ns;        // limit of the wait for the peers' gradients
};

// Signal buffer layout (32-bit words): ready[b][r] | done[b][r] | sumsq[b][r] (float bits)
__device__ __forceinline__ long long pad_ready(int nb, int b, int r) { return ((long long)b * kMaxRanks + r); }
__device__ __forceinline__ long long pad_done(int nb, int b, int r) { return ((long long)(nb + b) * kMaxRanks + r); }
__device__ __forceinline__ long long pad_sumsq(int nb, int b, int r) { return ((long long)(2 * nb + b) * kMaxRanks + r); }

template <bool NVLS>
__global__ void __launch_bounds__(kDpThreads)
dp_allreduce_kernel(const DpArgs a) {
  __shared__ float scratch[33];
  __shared__ int s_ok;
  __shared__ unsigned int s_last;
  const int nb = a.num_buckets, b = a.bucket;
  uint32_t* my_pad = a.pads[a.rank];
  const uint32_t e = a.epochs[b] + 1;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < a.world) {
    // Tell every rank that this rank's gradients of bucket b are final (redundant across CTAs: same value).
    __threadfence_system();
    st_release_sys(a.pads[threadIdx.x] + pad_ready(nb, b, a.rank), e);
    if (!wait_flag_ge(my_pad + pad_ready(nb, b, threadIdx.x), e, a.wait_ns)) s_ok = 0;
  }
  __syncthreads();
  float sq = 0.0f;
  if (s_ok) {
    // Slice owned by this rank, in 8-element (16-byte) vectors.
    const long long nvec = a.n / 8;
    const long long per = (nvec + a.world - 1) / a.world;
    const long long v0 = per * a.rank;
    const long long v1 = v0 + per < nvec ? v0 + per : nvec;
    const float inv = 1.0f / (float)a.world;
    // Four 16-byte vectors per thread and iteration: all four remote loads are issued before the first is used, so
    // a thread keeps 64 bytes in flight across the NVLink round trip instead of 16.
    constexpr int kUnroll = 4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long vb = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; vb < v1; vb += stride * kUnroll) {
      float f[kUnroll][8];
      bool live[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long v = vb + u * stride;
        live[u] = v < v1;
        const long long off = a.start + (live[u] ? v : vb) * 8;
        if (NVLS) {
          const uint4 q = multimem_ld_reduce_bf16x8(a.mc_base + off);
          const float2 p0 = unpack_bf16x2(q.x), p1 = unpack_bf16x2(q.y), p2 = unpack_bf16x2(q.z), p3 = unpack_bf16x2(q.w);
          f[u][0] = p0.x; f[u][1] = p0.y; f[u][2] = p1.x; f[u][3] = p1.y;
          f[u][4] = p2.x; f[u][5] = p2.y; f[u][6] = p3.x; f[u][7] = p3.y;
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) f[u][i] = 0.0f;
          for (int r = 0; r < a.world; ++r) {
            const uint4 q = ld_cg_v4(a.bases[r] + off);
            const float2 p0 = unpack_bf16x2(q.x), p1 = unpack_bf16x2(q.y), p2 = unpack_bf16x2(q.z), p3 = unpack_bf16x2(q.w);
            f[u][0] += p0.x; f[u][1] += p0.y; f[u][2] += p1.x; f[u][3] += p1.y;
            f[u][4] += p2.x; f[u][5] += p2.y; f[u][6] += p3.x; f[u][7] += p3.y;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (!live[u]) continue;
        const long long off = a.start + (vb + u * stride) * 8;
        uint4 o;
        o.x = pack_bf16x2(f[u][0] * inv, f[u][1] * inv);
        o.y = pack_bf16x2(f[u][2] * inv, f[u][3] * inv);
        o.z = pack_bf16x2(f[u][4] * inv, f[u][5] * inv);
        o.w = pack_bf16x2(f[u][6] * inv, f[u][7] * inv);
        // Sum of squares of the values every rank will hold (after bf16 rounding).
        const float2 q0 = unpack_bf16x2(o.x), q1 = unpack_bf16x2(o.y), q2 = unpack_bf16x2(o.z), q3 = unpack_bf16x2(o.w);
        sq += q0.x * q0.x + q0.y * q0.y + q1.x * q1.x + q1.y * q1.y + q2.x * q2.x + q2.y * q2.y + q3.x * q3.x + q3.y * q3.y;
        if (NVLS) {
          multimem_st_bf16x8(a.mc_base + off, o);
        } else {
          for (int r = 0; r < a.world; ++r) st_cg_v4(a.bases[r] + off, o);
        }
      }
    }
  }
  __threadfence_system();  // this thread's slice writes are visible system-wide before the CTA reports
  if (!s_ok && threadIdx.x == 0) sq = NAN;  // the owned slice was not averaged: poison the norm instead of hiding it
  sq = block_sum(sq, scratch);
  if (threadIdx.x == 0) {
    a.cta_partial[blockIdx.x] = sq;
    __threadfence_system();
    s_last = atomicAdd(a.cta_counter, 1u) == gridDim.x - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    // Last CTA of this rank: every slice write of this rank has been issued and fenced.
    __threadfence_system();
    float tot = 0.0f;
    if (threadIdx.x == 0) {
      for (unsigned i = 0; i < gridDim.x; ++i) tot += __ldcg(a.cta_partial + i);
      *a.cta_counter = 0;
      a.epochs[b] = e;
    }
    tot = __shfl_sync(0xffffffffu, tot, 0);
    if (threadIdx.x < a.world) {
      uint32_t* pad = a.pads[threadIdx.x];
      pad[pad_sumsq(nb, b, a.rank)] = __float_as_uint(tot);
      __threadfence_system();
      st_release_sys(pad + pad_done(nb, b, a.rank), e);
    }
  }
}

// One CTA: wait for every (bucket, rank) of this step, fold the sums of squares, write the clip control block.
__global__ void __launch_bounds__(256)
dp_finalize_kernel(const uint32_t* pad, const unsigned int* epochs, int num_buckets, int world, float max_norm,
                   float* ctrl, unsigned long long wait_ns) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const int total = num_buckets * world;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int b = i / world, r = i % world;
    if (!wait_flag_ge(pad + pad_done(num_buckets, b, r), epochs[b], wait_ns)) s_ok = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.0f;
    for (int b = 0; b < num_buckets; ++b)
      for (int r = 0; r < world; ++r) s += __uint_as_float(ld_acquire_sys(pad + pad_sumsq(num_buckets, b, r)));
    if (!s_ok) s = NAN;
    const float total_norm = sqrtf(s);
    const bool finite = isfinite(total_norm);
    float scale = 1.0f;
    if (finite && max_norm > 0.0f && total_norm > max_norm) scale = max_norm / total_norm;
    ctrl[0] = total_norm;
    ctrl[1] = scale;
    ctrl[2] = finite ? 1.0f : 0.0f;
    ctrl[3] = s;
  }
}

// Flat copy with eight 16-byte loads in flight per thread: a probe of what plain loads from a peer's memory (or from
// local memory) sustain, used as the link-bandwidth denominator of the fused-path reports.
__global__ void __launch_bounds__(kDpThreads)
copy_flat_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long nvec) {
  constexpr int kUnroll = 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long vb = (long long)blockIdx.x * blockDim.x + threadIdx.x; vb < nvec; vb += stride * kUnroll) {
    uint4 t[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long v = vb + u * stride;
      t[u] = ld_cg_v4(src + (v < nvec ? v : vb));
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long v = vb + u * stride;
      if (v < nvec) st_cg_v4(dst + v, t[u]);
    }
  }
}

}  // namespace dptb

using namespace dptb;

// dst[0, nbytes) = src[0, nbytes); both 16-byte aligned, nbytes a multiple of 16; either may be peer-mapped memory.
extern "C" int dptb_copy_flat(const void* src, void* dst, long long nbytes, int grid, void* stream) {
  if (nbytes <= 0) return 0;
  if ((nbytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return kErrBadShape;
  if (grid <= 0) grid = 4 * sm_count();
  copy_flat_kernel<<<grid, kDpThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), nbytes / 16);
  return counted(1, (int)cudaGetLastError());
}

struct DptbDpArgs {
  void* bases[kMaxRanks];
  void* pads[kMaxRanks];
  void* mc_base;
  int rank, world, bucket, num_buckets;
  long long start, n;
  float* cta_partial;
  unsigned int* cta_counter;
  unsigned int* epochs;
  int grid;
  int use_nvls;
  long long wait_ns;   // <= 0: the default limit of a wait
};

// Words a signal buffer needs for `num_buckets` buckets.
extern "C" long long dptb_dp_pad_words(int num_buckets) { return 3LL * num_buckets * kMaxRanks; }

extern "C" int dptb_dp_allreduce(const DptbDpArgs* h, void* stream) {
  auto st = static_cast<cudaStream_t>(stream);
  if (h->world < 1 || h->world > kMaxRanks || h->rank < 0 || h->rank >= h->world) return kErrBadShape;
  if (h->n <= 0) return 0;
  if ((h->n % 8) || (h->start % 8) || h->grid < 1) return kErrBadShape;
  DpArgs a;
  for (int r = 0; r < kMaxRanks; ++r) {
    a.bases[r] = static_cast<__nv_bfloat16*>(h->bases[r]);
    a.pads[r] = static_cast<uint32_t*>(h->pads[r]);
  }
  a.mc_base = static_cast<__nv_bfloat16*>(h->mc_base);
  a.rank = h->rank; a.world = h->world; a.bucket = h->bucket; a.num_buckets = h->num_buckets;
  a.start = h->start; a.n = h->n;
  a.cta_partial = h->cta_partial; a.cta_counter = h->cta_counter; a.epochs = h->epochs;
  a.wait_ns = h->wait_ns > 0 ? (unsigned long long)h->wait_ns : kWaitLimitNs;
  if (h->use_nvls && a.mc_base) dp_allreduce_kernel<true><<<h->grid, kDpThreads, 0, st>>>(a);
  else                          dp_allreduce_kernel<false><<<h->grid, kDpThreads, 0, st>>>(a);
  return counted(1, (int)cudaGetLastError());
}

extern "C" int dptb_dp_finalize(const void* pad, const unsigned int* epochs, int num_buckets, int world,
                                float max_norm, float* ctrl, long long wait_ns, void* stream) {
  dp_finalize_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(pad), epochs, num_buckets, world, max_norm, ctrl,
      wait_ns > 0 ? (unsigned long long)wait_ns : kWaitLimitNs);
  return counted(1, (int)cudaGetLastError());
}
