// Column-sum entry point that allocates nothing.  It has no counterpart in the reference library: the reference
// allocates two device buffers inside every native call (lib/native/src/engine.cu:24-59).
//
// Who needs it: code that must not call cudaMalloc while it runs -- a caller inside a CUDA-graph capture or a
// latency-critical serving loop where an allocation would synchronise the device, a plug-in loaded by a host
// application that owns the memory pool, or a process that has handed all device memory to another allocator.
// dptb_colsum (csrc/elementwise.cu) makes such callers bring an fp32 scratch buffer; this variant keeps the scratch in
// a fixed array inside the library instead, so the caller passes only its input and output.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest number of columns one call may reduce.  The scratch array holds DPTB_COLSUM_STATIC_PARTS partial rows of this
// many floats: 32 x 8192 x 4 bytes = 1 MiB of device memory on every GPU that loads the library, until the process exits.
#define DPTB_COLSUM_STATIC_MAX_COLS 8192
#define DPTB_COLSUM_STATIC_PARTS 32

// out[c] (+)= sum over rows of x[r * ld + c], for c < cols.
//   x      device pointer, rows x cols with leading dimension ld (elements); dtype 0 = fp32, 1 = bf16
//   out    device pointer, cols elements of the same dtype; accumulate != 0 adds to what is there
//   stream CUDA stream to launch on (0 = the default stream)
// Returns 0 on success, a positive cudaError_t if a runtime call failed, -4 if cols > DPTB_COLSUM_STATIC_MAX_COLS (nothing
// is launched), -1 for other bad arguments.
//
// The first call on each device looks up the device address of the scratch array (cudaGetSymbolAddress, with that
// device current); make that first call before any stream capture begins.  No call allocates or frees memory.
// All calls on a device share the one scratch array: two calls whose kernels overlap on the GPU (different streams
// without an ordering between them) race on it.  Calls on one stream, or ordered by events, are safe.  The array
// keeps the previous call's partial sums; nothing in it has to start at zero, because every partial that a call reads
// is first written by that call.
int dptb_colsum_static(const void* x, long long ld, void* out, long long rows, int cols, int accumulate, int dtype,
                       void* stream);

#ifdef __cplusplus
}
#endif
