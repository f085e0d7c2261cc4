// Host-side helpers shared by the launchers: error codes, TMA tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda), device properties.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace dptb {

// Return codes of every extern "C" entry point: 0 = ok, > 0 = cudaError_t, < 0 = library error.
enum HostError : int {
  kErrBadShape = -1,      // shape / stride / alignment the kernel cannot take
  kErrNoDriver = -2,      // cuTensorMapEncodeTiled could not be resolved
  kErrTensorMap = -3,     // the driver rejected a tensor map
  kErrTooLarge = -4,      // a fixed-capacity scratch area is too small for this call
  kErrUnsupported = -5,
};

#define DPTB_CUDA_OK(expr)                     \
  do {                                         \
    cudaError_t _e = (expr);                   \
    if (_e != cudaSuccess) return (int)_e;     \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// 2-D bf16 tensor map with 128-byte swizzle.  `inner` is the contiguous extent (elements), `outer` the number of rows,
// `row_stride_bytes` the distance between rows (multiple of 16).  Out-of-range reads give zeros.
inline int encode_tmap_2d_bf16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                               uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_tiled();
  if (!fn) return kErrNoDriver;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) || box_inner * 2 > 128 || box_outer > 256)
    return kErrBadShape;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : kErrTensorMap;
}

// Rank-N (N <= 5) bf16 tensor map with 128-byte swizzle: dims[0] is contiguous; strides[i] (bytes) is the stride of
// dims[i+1].  The rank must equal the dimensionality of the copy instruction that uses the map.
inline int encode_tmap_nd_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims_in,
                               const uint64_t* strides_bytes, const uint32_t* box_in) {
  EncodeTiledFn fn = get_encode_tiled();
  if (!fn) return kErrNoDriver;
  if (rank < 1 || rank > 5 || (reinterpret_cast<uintptr_t>(base) & 15)) return kErrBadShape;
  cuuint64_t dims[5];
  cuuint64_t strides[4];
  cuuint32_t box[5];
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    dims[i] = dims_in[i];
    box[i] = box_in[i];
  }
  for (int i = 0; i + 1 < rank; ++i) {
    if (strides_bytes[i] & 15) return kErrBadShape;
    strides[i] = strides_bytes[i];
  }
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : kErrTensorMap;
}

// Number of kernels this library has launched since the last reset (host-side bookkeeping for benchmarks).
inline long long& launch_counter() {
  static long long count = 0;
  return count;
}
inline int counted(int kernels, int rc) {
  if (rc == 0) launch_counter() += kernels;
  return rc;
}

inline int sm_count() {
  static int cached[16] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Whether the kernels that support it are launched as programmatic dependents of their predecessor on the stream
// (see pdl_wait below).  Off by default; the tensor-parallel decode engine turns it on around its step.
inline int& pdl_flag() {
  static int on = 0;
  return on;
}

#ifdef __CUDACC__
// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization attribute may start
// while its predecessor on the stream is still running: everything it does before pdl_wait() (barrier set-up, TMEM
// allocation, loads of data the predecessor does not write) overlaps the predecessor's tail; pdl_wait() returns once
// the predecessor has completed and its writes are visible.  pdl_launch_dependents() in the predecessor lets such a
// dependent start early.  Both are no-ops in launches without the attribute / without such a dependent.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Launches `kern`, as a programmatic dependent of the previous kernel on the stream when pdl_flag() is set.  Such a
// kernel calls pdl_wait() before its first global access and pdl_launch_dependents() after it, never before: the kernel
// after it must not start while the kernel two places back is still running.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  if (!pdl_flag()) {
    kern<<<grid, block, smem, st>>>(args...);
    return cudaGetLastError();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

}  // namespace dptb
