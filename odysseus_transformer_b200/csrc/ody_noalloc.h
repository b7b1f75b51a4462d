// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (which has no native code and lets PyTorch
// allocate every temporary).  It exists for hosts that drive these kernels from a place where a device
// allocation is off the table: a runtime that sized all of its memory up front and owns no allocator,
// a step running under a fixed memory budget where a cudaMalloc would also stall the device, or a
// plain C caller that has the input and output buffers and nothing else.
//
// It computes exactly what ody_rmsnorm_bwd computes, but the cross-block partial sums of dw live in
// a scratch array that is part of the loaded library (file-scope __device__ storage,
// ODY_NOALLOC_RMSNORM_SCRATCH_BYTES per GPU that loads it, held until the process exits) instead of a
// caller-provided workspace.  The call itself performs no cudaMalloc / cudaFree and uses no allocating
// library routine.
//
// Limits and rules:
//   * dim must be a multiple of 8 and at most ODY_NOALLOC_RMSNORM_MAX_DIM; larger sizes are refused
//     with ODY_NOALLOC_ERR_TOO_LARGE before anything is launched (ody_noalloc_strerror explains codes).
//   * Pointers: dy, x, w, dx (and ds when given) must be non-null device pointers aligned to 16 bytes, rstd and dw
//     non-null and aligned to 4 bytes (rows are dim * 2 bytes apart with dim a multiple of 8, so every row then
//     starts on a 16-byte boundary too).  Anything else is refused with ODY_NOALLOC_ERR_BAD_POINTER before a
//     launch - the kernels use 16-byte accesses and would otherwise fault on the device.  With rows == 0 only dw
//     is touched (set to zero); the other pointers may then be null.
//   * The first call on each device looks up the scratch array's device address (one
//     cudaGetSymbolAddress with that device current).  Make that first call outside of any stream
//     capture; later calls only launch kernels.
//   * All calls on a device share the one scratch array.  Nothing in it has to start at zero - every
//     launch overwrites the part it then reads - but two calls whose kernels overlap on the GPU
//     (different streams, no ordering between them) race on it.  Order them on one stream or with events.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define ODY_NOALLOC_RMSNORM_MAX_DIM 8192
#define ODY_NOALLOC_RMSNORM_MAX_BLOCKS 148
#define ODY_NOALLOC_RMSNORM_SCRATCH_BYTES (ODY_NOALLOC_RMSNORM_MAX_BLOCKS * ODY_NOALLOC_RMSNORM_MAX_DIM * 4)
#define ODY_NOALLOC_ERR_TOO_LARGE 9001
#define ODY_NOALLOC_ERR_BAD_SHAPE 9002
#define ODY_NOALLOC_ERR_BAD_POINTER 9003

#ifdef __cplusplus
extern "C" {
#endif

// dy, x [rows, dim] bf16; w [dim] bf16; rstd [rows] fp32; ds [rows, dim] bf16 or NULL (added to dx);
// outputs dx [rows, dim] bf16 and dw [dim] fp32.  Returns 0, a cudaError_t value, or an ODY_NOALLOC_ERR_* code.
int ody_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* ds, void* dx,
                            float* dw, int64_t rows, int dim, cudaStream_t stream);

// Human-readable text for a return value of the function above.
const char* ody_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
