// ody_rmsnorm_bwd_noalloc: RMSNorm backward whose dw partial sums use library-owned device storage.
// See ody_noalloc.h for who needs this and the rules that come with it.
#include <mutex>

#include "common.cuh"
#include "ody_noalloc.h"

namespace ody {
namespace noalloc {

// One slab per GPU that loads this library: [MAX_BLOCKS][MAX_DIM] fp32 partial sums of dw.
static __device__ __align__(256) float g_dw_partial[ODY_NOALLOC_RMSNORM_MAX_BLOCKS * ODY_NOALLOC_RMSNORM_MAX_DIM];

constexpr int kMaxDevices = 64;
static float* g_scratch_addr[kMaxDevices] = {};   // device address of g_dw_partial, per device
static std::mutex g_mu;

// Same arithmetic as rmsnorm_bwd_k in elementwise.cu; each block walks rows blockIdx.x, +gridDim.x, ...
// and leaves its column sums of dy * xhat in partial[blockIdx.x][:].
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_bwd_fixed_k(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                           const bf16* __restrict__ w, const float* __restrict__ rstd,
                                                           const bf16* __restrict__ ds, bf16* __restrict__ dx,
                                                           float* __restrict__ partial, int64_t rows, int dim) {
  __shared__ float red[33];
  float wv[NV][8], acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    if (c < dim) unpack8(ld8(w + c), wv[i]);
  }
  const float inv_dim = 1.f / (float)dim;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rs = rstd[row];
    float g[NV][8], xh[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (threadIdx.x + i * blockDim.x) * 8;
      if (c < dim) {
        float a[8];
        unpack8(ld8(dy + row * dim + c), a);
        unpack8(ld8(x + row * dim + c), xh[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rs;
          acc[i][j] += a[j] * xh[i][j];
          g[i][j] = a[j] * wv[i][j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    dot = block_sum(dot, red) * inv_dim;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (threadIdx.x + i * blockDim.x) * 8;
      if (c < dim) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (g[i][j] - xh[i][j] * dot) * rs;
        if (ds != nullptr) {
          float s[8];
          unpack8(ld8(ds + row * dim + c), s);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += s[j];
        }
        st8(dx + row * dim + c, pack8(o));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 8;
    if (c < dim) {
      float* p = partial + (int64_t)blockIdx.x * dim + c;
      *reinterpret_cast<float4*>(p) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
  }
}

__global__ void colsum_fixed_k(const float* __restrict__ partial, float* __restrict__ out, int nblocks, int dim) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= dim) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[(int64_t)b * dim + c];
  out[c] = s;
}

// Device address of the scratch slab for the CURRENT device.  In host code the name g_dw_partial is only
// a handle for the symbol, never a pointer a kernel may use; the real address comes from the runtime.
static int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_dw_partial);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return (int)cudaErrorInvalidSymbol;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace noalloc
}  // namespace ody

extern "C" int ody_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* ds,
                                       void* dx, float* dw, int64_t rows, int dim, cudaStream_t stream) {
  using namespace ody;
  using namespace ody::noalloc;
  if (rows < 0 || dim <= 0 || (dim % 8) != 0) return ODY_NOALLOC_ERR_BAD_SHAPE;
  if (dim > ODY_NOALLOC_RMSNORM_MAX_DIM) return ODY_NOALLOC_ERR_TOO_LARGE;
  // the kernels move 16 bytes per access on dy / x / w / ds / dx and 4 on rstd / dw: a null or misaligned pointer
  // would fault on the device, so it is refused here instead
  if (dw == nullptr || ((uintptr_t)dw & 3)) return ODY_NOALLOC_ERR_BAD_POINTER;
  if (rows > 0) {
    if (dy == nullptr || x == nullptr || w == nullptr || rstd == nullptr || dx == nullptr) return ODY_NOALLOC_ERR_BAD_POINTER;
    if ((((uintptr_t)dy | (uintptr_t)x | (uintptr_t)w | (uintptr_t)dx | (uintptr_t)ds) & 15) || ((uintptr_t)rstd & 3))
      return ODY_NOALLOC_ERR_BAD_POINTER;
  } else {
    // no rows: the sum over nothing.  dw is cleared with a plain asynchronous memset; nothing else is touched.
    return (int)cudaMemsetAsync(dw, 0, (size_t)dim * sizeof(float), stream);
  }
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  const int nb = (int)(rows < ODY_NOALLOC_RMSNORM_MAX_BLOCKS ? (rows > 0 ? rows : 1) : ODY_NOALLOC_RMSNORM_MAX_BLOCKS);
  const int nv = (dim + 2047) / 2048;
#define ODY_L(NV)                                                                                                   \
  rmsnorm_bwd_fixed_k<NV><<<nb, 256, 0, stream>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)ds, \
                                                  (bf16*)dx, scratch, rows, dim)
  if (nv <= 1) ODY_L(1); else if (nv <= 2) ODY_L(2); else ODY_L(4);
#undef ODY_L
  colsum_fixed_k<<<(dim + 255) / 256, 256, 0, stream>>>(scratch, dw, nb, dim);
  return (int)cudaGetLastError();
}

extern "C" const char* ody_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "success";
    case ODY_NOALLOC_ERR_TOO_LARGE:
      return "ody_rmsnorm_bwd_noalloc: dim exceeds ODY_NOALLOC_RMSNORM_MAX_DIM (8192); the built-in scratch array cannot hold it";
    case ODY_NOALLOC_ERR_BAD_SHAPE:
      return "ody_rmsnorm_bwd_noalloc: rows must be >= 0 and dim a positive multiple of 8";
    case ODY_NOALLOC_ERR_BAD_POINTER:
      return "ody_rmsnorm_bwd_noalloc: dy, x, w, dx (and ds when given) must be non-null and 16-byte aligned; rstd and dw "
             "non-null and 4-byte aligned";
    default: return cudaGetErrorString((cudaError_t)code);
  }
}
