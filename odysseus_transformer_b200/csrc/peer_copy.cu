// Plain peer-memory copy kernel: 16-byte loads and stores issued by every thread, 8 in flight per thread.
// Used to move a buffer to or from another GPU's symmetric memory inside a stream (no library call),
// and by benchmarks/p2p_bench.py to measure what NVLink gives per SM for pushes and pulls.
#include <cuda_runtime.h>
#include <stdint.h>

#include "ody_kernels.h"

namespace ody {

__global__ void peer_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, int64_t nvec) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (i0 + u * stride < nvec) v[u] = src[i0 + u * stride];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (i0 + u * stride < nvec) dst[i0 + u * stride] = v[u];
  }
}

}  // namespace ody

extern "C" int ody_peer_copy(void* dst, const void* src, int64_t bytes, int n_ctas, int threads, cudaStream_t st) {
  if ((bytes % 16) || (((uintptr_t)dst | (uintptr_t)src) & 15) || n_ctas <= 0 || threads <= 0 || threads > 1024)
    return (int)cudaErrorInvalidValue;
  if (bytes == 0) return 0;
  ody::peer_copy_kernel<<<n_ctas, threads, 0, st>>>((uint4*)dst, (const uint4*)src, bytes / 16);
  return (int)cudaGetLastError();
}
