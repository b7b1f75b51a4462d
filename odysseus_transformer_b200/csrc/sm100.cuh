// Thin inline-PTX wrappers for the Blackwell (sm_100a) execution model: mbarrier, TMA
// (cp.async.bulk.tensor, never with cluster multicast), tcgen05 MMA / TMEM, plus host-side tensor-map
// encoding.  Every wait is bounded: it gives up after ~1 s of SM clocks or as soon as the CTA-wide
// abort flag is raised, so a protocol bug ends in an error code instead of a hung GPU.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ody {

// ------------------------------------------------------------------------------------------- error codes
enum : int {
  ODY_OK = 0,
  ODY_ERR_TIMEOUT_FULL = 101,     // consumer waited for TMA data that never arrived
  ODY_ERR_TIMEOUT_EMPTY = 102,    // producer waited for a free smem stage
  ODY_ERR_TIMEOUT_TMEM_FULL = 103,
  ODY_ERR_TIMEOUT_TMEM_EMPTY = 104,
  ODY_ERR_TIMEOUT_PEER = 105,     // a flag owned by another GPU was never set
  ODY_ERR_TIMEOUT_MISC = 106,
};

#ifdef __CUDACC__

#ifndef ODY_SPIN_LIMIT_CYCLES
#define ODY_SPIN_LIMIT_CYCLES (2000000000ll)   // ~1 s at B200 clocks
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  `abort_flag` is a CTA-wide shared word: once any thread sets it every waiter leaves.
// Returns true when the phase completed; on timeout records `code` in *err (global, first error wins),
// raises the abort flag and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
#ifdef ODY_WAIT_SLEEP_NS
    __nanosleep(ODY_WAIT_SLEEP_NS);     // a polling warp otherwise competes for issue slots with the working warps of its scheduler
#endif
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > ODY_SPIN_LIMIT_CYCLES) {
        if (err != nullptr) atomicCAS(err, 0, code);
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// ---- TMA (2-D tiles).  Loads complete on an mbarrier; stores use bulk groups.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* tmap, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(tmap), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tmap, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(tmap), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

__device__ __forceinline__ void named_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// Named barrier that also ANDs a predicate over its participants: used so that the warps sharing a barrier
// leave a loop together when one of them saw a wait give up (a warp that left alone would strand the others).
// ---- exponentials for the attention kernels
// exp2_mufu is the special-function unit's ex2.  exp2_poly / exp2_poly2 evaluate 2^x on the FMA pipe instead:
// 2^x = 2^n * 2^f with n = round(x) taken from the mantissa of x + 1.5 * 2^23, f in [-0.5, 0.5], a degree-3 minimax
// polynomial for 2^f (relative error 7.5e-5, far below the bf16 rounding the probabilities get anyway) and n added
// to the exponent field.  Valid for x <= 127; x below -125 returns 2^-125.
__device__ __forceinline__ float exp2_mufu(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float exp2_poly(float x) {
  x = fmaxf(x, -125.f);
  const float t = x + 12582912.f;
  const float f = x - (t - 12582912.f);
  float p = fmaf(0.0551716499f, f, 0.2426111251f);
  p = fmaf(p, f, 0.6932609677f);
  p = fmaf(p, f, 0.9999280572f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
// Packed fp32 pairs (sm_100 executes add / mul / fma on two floats per instruction): the softmax warps are bound
// by instruction issue, so pairing halves the cost of their elementwise arithmetic.
__device__ __forceinline__ uint64_t pk2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ uint64_t pk2u(uint32_t a, uint32_t b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ void upk2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// 2^x for a packed pair on the FMA pipe (same scheme as exp2_poly): about 10 instructions per pair
__device__ __forceinline__ void exp2_poly2(uint64_t x2, float& r0, float& r1) {
  float x0, x1;
  upk2(x2, x0, x1);
  x2 = pk2(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
  const uint64_t magic = pk2(12582912.f, 12582912.f), nmagic = pk2(-12582912.f, -12582912.f);
  const uint64_t t2 = add2(x2, magic);
  const uint64_t f2 = fma2(add2(t2, nmagic), pk2(-1.f, -1.f), x2);      // x - round(x), in [-0.5, 0.5]
  uint64_t p2 = fma2(pk2(0.0551716499f, 0.0551716499f), f2, pk2(0.2426111251f, 0.2426111251f));
  p2 = fma2(p2, f2, pk2(0.6932609677f, 0.6932609677f));
  p2 = fma2(p2, f2, pk2(0.9999280572f, 0.9999280572f));
  float p0, p1, t0, t1;
  upk2(p2, p0, p1);
  upk2(t2, t0, t1);
  r0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  r1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

// Warpgroup register reallocation (all four warps of an aligned warpgroup execute the same instruction):
// producer / issuer warpgroups give registers away, the math warpgroups take them.
template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

__device__ __forceinline__ bool named_barrier_and(int id, int nthreads, bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, %2, %3, q;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(r)
      : "r"((uint32_t)ok), "r"(id), "r"(nthreads)
      : "memory");
  return r != 0;
}

// ---- tcgen05 / TMEM (cta_group::1)
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {        // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues.
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// mbarrier arrives once all tcgen05 ops issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane (base_lane + i), columns [c, c+32)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// ---- descriptors
// Shared-memory matrix descriptor, 128-byte swizzle (TMA SWIZZLE_128B tiles whose rows are 128 bytes).
//   K-major operand  : rows = M/N index, 64 bf16 of K per row; 8-row groups are `sbo` bytes apart (1024 when dense).
//   MN-major operand : rows = K index, 64 bf16 of M/N per row; 8-row K groups `sbo` apart, 64-element M/N blocks `lbo` apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version for sm_100
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}
// K-major operand stored as K / 16 slices of [rows x 32 B] with the 32-byte swizzle (TMA SWIZZLE_32B tiles whose rows are
// 32 bytes): the 16-deep slice one MMA instruction reads is then one contiguous rows x 32 B block - whole 128-byte
// lines - instead of a 32-byte piece out of every row of a 128-byte-swizzled tile.  8-row groups are 256 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_sw32(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
  d |= (uint64_t)(1) << 16;                  // leading-dimension offset: unused for swizzled K-major operands
  d |= (uint64_t)((256 >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version for sm_100
  d |= (uint64_t)6 << 61;   // SWIZZLE_32B
  return d;
}
// Same, without swizzle ("interleaved" core matrices of 8 rows x 16 bytes): K-adjacent core matrices `lbo` bytes
// apart, 8-row groups `sbo` apart.  Used for the 16-column statistics tiles of the attention backward.
__device__ __forceinline__ uint64_t make_smem_desc_noswizzle(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version for sm_100
  return d;
}
// Advance a descriptor's start address by `bytes` (a multiple of 16).  Only the low word changes - the issuing
// thread spends one add per MMA instead of rebuilding the descriptor, and a single thread's instruction
// stream is what bounds how fast small MMAs can be issued.
__device__ __forceinline__ uint64_t desc_advance(uint64_t d, uint32_t bytes) {
  uint2 v = *reinterpret_cast<uint2*>(&d);
  v.x += bytes >> 4;
  return *reinterpret_cast<uint64_t*>(&v);
}
// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ------------------------------------------------------------------------------------------- rotary embedding in a GEMM epilogue
// The output columns are heads of 128 in groups of `period_cols`; the first `rot_cols` columns of every group belong
// to heads that are rotated (q and k of a packed q|k|v projection), with the two halves of a head 64 columns apart.
// An epilogue thread owns one output row and takes the accumulator in chunks of 64 columns, so a chunk is one half of
// a head: it reads the other half (64 TMEM columns up or down) next to its own and writes
//   low half:  x_lo * cos - x_hi * sin        high half:  x_hi * cos + x_lo * sin
// with cos / sin [rows, 64] fp32 indexed by the output row.  cos == nullptr switches it off.
struct RopeEpi {
  const float* cos;
  const float* sin;
  int period_cols, rot_cols;
};
__device__ __forceinline__ bool rope_epi_wants(const RopeEpi& rp, int col0) {
  return rp.cos != nullptr && (col0 % rp.period_cols) < rp.rot_cols;
}
// v: this chunk's 64 accumulators (fp32 bits), w: the partner half's; hi: this chunk is the high half of its head
__device__ __forceinline__ void rope_epi_apply(const RopeEpi& rp, int64_t row, bool hi, uint32_t* v, const uint32_t* w) {
  const float4* c4 = reinterpret_cast<const float4*>(rp.cos + row * 64);
  const float4* s4 = reinterpret_cast<const float4*>(rp.sin + row * 64);
  const float sg = hi ? 1.f : -1.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float4 c = __ldg(c4 + i), s = __ldg(s4 + i);
    v[4 * i + 0] = __float_as_uint(__uint_as_float(v[4 * i + 0]) * c.x + sg * __uint_as_float(w[4 * i + 0]) * s.x);
    v[4 * i + 1] = __float_as_uint(__uint_as_float(v[4 * i + 1]) * c.y + sg * __uint_as_float(w[4 * i + 1]) * s.y);
    v[4 * i + 2] = __float_as_uint(__uint_as_float(v[4 * i + 2]) * c.z + sg * __uint_as_float(w[4 * i + 2]) * s.z);
    v[4 * i + 3] = __float_as_uint(__uint_as_float(v[4 * i + 3]) * c.w + sg * __uint_as_float(w[4 * i + 3]) * s.w);
  }
}

#endif  // __CUDACC__

// ------------------------------------------------------------------------------------------- host: tensor maps
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_fn() {
  static PFN_encodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (PFN_encodeTiled)p;
  }
  return fn;
}

// 2-D bf16 tensor, inner dim contiguous: dims {inner, outer}, row pitch in BYTES, box {box_inner, box_outer},
// 128-byte swizzle (box_inner * 2 bytes must be 128).  Returns 0 on success.
inline int make_tmap_2d_bf16(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_bytes,
                             uint32_t box_inner, uint32_t box_outer) {
  PFN_encodeTiled enc = get_encode_fn();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (int)r;
}

// MN-major operand [K rows][MN elements] viewed as {64 (mn), K, MN/64}: one box {64, box_k, nblk} lands in shared
// memory as nblk consecutive [box_k x 128 B] swizzled blocks - the layout tcgen05 wants for an MN-major tile -
// so a whole operand tile is ONE TMA instruction.  Needs MN % 64 == 0.
inline int make_tmap_mn_blocked_bf16(CUtensorMap* m, const void* base, uint64_t mn, uint64_t k, uint64_t pitch_bytes,
                                     uint32_t box_k, uint32_t nblk) {
  PFN_encodeTiled enc = get_encode_fn();
  if (enc == nullptr) return -1;
  cuuint64_t dims[3] = {64, k, mn / 64};
  cuuint64_t strides[2] = {pitch_bytes, 128};
  cuuint32_t box[3] = {64, box_k, nblk};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (int)r;
}

// Same, without swizzle: for plain copies, where the inner box may be up to 256 elements wide.
inline int make_tmap_2d_bf16_linear(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_bytes,
                                    uint32_t box_inner, uint32_t box_outer) {
  PFN_encodeTiled enc = get_encode_fn();
  if (enc == nullptr) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (int)r;
}

// 3-D bf16 tensor {inner, mid, outer} with byte pitches for mid and outer.  box_inner * 2 bytes must equal the swizzle
// span: 128 for the default, 32 with sw32 (box_inner 16).
inline int make_tmap_3d_bf16(CUtensorMap* m, const void* base, uint64_t inner, uint64_t mid, uint64_t outer,
                             uint64_t pitch_mid_bytes, uint64_t pitch_outer_bytes, uint32_t box_inner,
                             uint32_t box_mid, uint32_t box_outer, bool sw32 = false) {
  PFN_encodeTiled enc = get_encode_fn();
  if (enc == nullptr) return -1;
  cuuint64_t dims[3] = {inner, mid, outer};
  cuuint64_t strides[2] = {pitch_mid_bytes, pitch_outer_bytes};
  cuuint32_t box[3] = {box_inner, box_mid, box_outer};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (int)r;
}

}  // namespace ody
