// Allocation-free column sum: the two-stage deterministic reduction of dptb_colsum with its partial-sum scratch held
// in a fixed device array of this file instead of a caller-provided buffer.  See colsum_static.h for the contract.
#include "colsum_static.h"

#include <atomic>

#include "common/host.h"
#include "common/reduce.cuh"

namespace {

// Partial sums [DPTB_COLSUM_STATIC_PARTS][cols] of the call in flight.  In host code this name is only a handle for
// cudaGetSymbolAddress; device code uses it directly.
static __device__ __align__(256) float g_colsum_scratch[DPTB_COLSUM_STATIC_PARTS * DPTB_COLSUM_STATIC_MAX_COLS];

// Stage 1: block = 32 lanes x 2 adjacent columns, 8 row lanes; gridDim.y = DPTB_COLSUM_STATIC_PARTS row slices.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_static_partial_kernel(const T* __restrict__ x, long long ld, long long rows, int cols, float* __restrict__ partial) {
  __shared__ float sm[8][65];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 64 + cx * 2;
  float s0 = 0.0f, s1 = 0.0f;
  if (c < cols) {
    const long long step = (long long)gridDim.y * 8;
    for (long long r = (long long)blockIdx.y * 8 + ry; r < rows; r += step) {
      s0 += dptb::to_f32(x[r * ld + c]);
      if (c + 1 < cols) s1 += dptb::to_f32(x[r * ld + c + 1]);
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

// Stage 2: fold the row slices in slice order.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_static_final_kernel(const float* __restrict__ partial, int nparts, int cols, T* __restrict__ out, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.0f;
  for (int p = 0; p < nparts; ++p) s += partial[(long long)p * cols + c];
  if (accumulate) s += dptb::to_f32(out[c]);
  out[c] = dptb::from_f32<T>(s);
}

// Device address of g_colsum_scratch on the current device, resolved once per device.
int scratch_for_current_device(float** out) {
  // Host threads may make their first calls at the same time: the slots are atomics, and two threads that both find a
  // slot empty both resolve the same address and store the same value.
  static std::atomic<float*> cached[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return dptb::kErrBadShape;
  float* p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_colsum_scratch);
    if (e != cudaSuccess) return (int)e;
    cached[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return 0;
}

}  // namespace

extern "C" int dptb_colsum_static(const void* x, long long ld, void* out, long long rows, int cols, int accumulate,
                                  int dtype, void* stream) {
  if (cols <= 0) return 0;
  if (cols > DPTB_COLSUM_STATIC_MAX_COLS) {
    fprintf(stderr, "dptb_colsum_static: cols = %d exceeds the fixed scratch capacity of %d columns\n", cols,
            DPTB_COLSUM_STATIC_MAX_COLS);
    return dptb::kErrTooLarge;
  }
  if (!x || !out || rows < 0 || ld < cols || (dtype != 0 && dtype != 1)) return dptb::kErrBadShape;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  auto st = static_cast<cudaStream_t>(stream);
  const int nparts = DPTB_COLSUM_STATIC_PARTS;
  dim3 grid((cols + 63) / 64, nparts);
  if (dtype) colsum_static_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ld, rows, cols, scratch);
  else       colsum_static_partial_kernel<float><<<grid, 256, 0, st>>>((const float*)x, ld, rows, cols, scratch);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return dptb::counted(0, (int)e);
  if (dtype) colsum_static_final_kernel<__nv_bfloat16><<<(cols + 255) / 256, 256, 0, st>>>(scratch, nparts, cols, (__nv_bfloat16*)out, accumulate);
  else       colsum_static_final_kernel<float><<<(cols + 255) / 256, 256, 0, st>>>(scratch, nparts, cols, (float*)out, accumulate);
  return dptb::counted(2, (int)cudaGetLastError());
}
