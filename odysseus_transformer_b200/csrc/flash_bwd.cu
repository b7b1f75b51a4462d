// Attention backward for sm_100a (head_dim 128, bf16, GQA): dQ, dK, dV from (dO, Q, K, V, O, LSE).
//
// The reference gets this from flash_attn_2_cuda.bwd through autograd (reference
// decoder/odysseus.py:256-263; its ring dependency calls the same kernel per block).  Here it is three
// kernels built on tcgen05 / TMEM / TMA:
//
//   prep   : -delta[h,t] = -sum_d dO*O, and -LSE in the exp2 domain (negated so the kernels can fuse them into packed
//            fma / add instructions), both padded to 128 rows.
//   dkdv   : one CTA per (128-row KV tile, kv head).  K and V stay in shared memory; 128-row blocks of Q
//            and dO stream through two TMA rings.  S^T = K Q^T and dP^T = V dO^T land in TMEM (kv rows on
//            lanes), eight warps (two per lane quarter, 64 columns each) turn them into P^T and dS^T (bf16,
//            written back over the same TMEM columns) and the tensor core accumulates dV += P^T dO,
//            dK += dS^T Q in TMEM (128 + 128 + 128 + 128 = 512 columns).  Every tcgen05.mma is 128x128x16:
//            a single thread issues one instruction per ~80 cycles whatever its shape, so 64-wide blocks
//            would leave the tensor core half idle.  S^T / dP^T are single buffered; the issue order
//            dV(i), S^T(i+1), dK(i), dP^T(i+1) keeps the in-order tensor pipe busy while the softmax warps
//            work on the other matrix.  Query heads sharing the kv head are looped inside.
//   dq     : one CTA per (128-row query tile, head).  Q and dO stay in shared memory; 128-row blocks of K
//            and V stream.  S = Q K^T, dP = dO V^T (double buffered), dS (bf16 in TMEM) and dQ += dS K.
//
// Splitting dQ from dK/dV recomputes S and dP once more but needs no atomics and is deterministic.
// Gradients are written with TMA stores through row-pitched tensor maps, so dq/dk/dv may be slices
// of one packed [T, hq + 2 hkv, 128] gradient tensor.
#include "ody_kernels.h"
#include "sm100.cuh"

// Of every ODY_BWD_POLY_DEN column pairs, the first ODY_BWD_POLY_NUM take their exponentials on the FMA pipe
// (exp2_poly2) instead of the special-function unit.  Measured on B200: any mix is a few percent slower than
// all-MUFU - the softmax warps are bound by the latency of their dependent chains, not by either pipe - so it is off.
#ifndef ODY_BWD_POLY_NUM
#define ODY_BWD_POLY_NUM 0
#define ODY_BWD_POLY_DEN 2
#endif

namespace ody {
namespace bwd {

constexpr int HD = 128;
constexpr int BIG = 128;                         // resident tile rows
constexpr int BLK = 128;                         // streamed block rows
constexpr int BIG_BYTES = BIG * HD * 2;          // 32 KB (two halves of [128 x 128 B])
constexpr int BIG_HALF = BIG_BYTES / 2;
constexpr int BLK_BYTES = BLK * HD * 2;          // 32 KB (two halves of [128 x 128 B])
constexpr int BLK_HALF = BLK_BYTES / 2;
constexpr int STAGES = 2;
constexpr int STAT_TILE = BLK * 32;              // one statistics tile: 128 rows x 16 bf16, no swizzle (see prep_kernel)
constexpr int STAT_BYTES = 2 * STAT_TILE;        // -lse/scale tile and -delta tile of one streamed block
// warps 0..3: TMA producer, MMA issuer, two idle (they complete the warpgroup whose registers are given away);
// warps 4..11: softmax / epilogue, two per TMEM lane quarter
constexpr int NUM_THREADS = 384;
// Register split by setmaxnreg.  A CTA of 384 threads is launched with 168 registers per thread (65536 / 384,
// rounded down to a multiple of 8); the split must fit inside THAT allocation or the increase never returns.
constexpr int REGS_LAUNCH = 168, REGS_ISSUE = 72, REGS_MATH = 216;
static_assert(128 * REGS_ISSUE + 256 * REGS_MATH <= NUM_THREADS * REGS_LAUNCH, "setmaxnreg split exceeds the CTA's registers");
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ------------------------------------------------------------------------------------------- prep
// delta_pad / lse2_pad: [H, Tpad] fp32 holding -delta and -lse * log2(e); Tpad multiple of 128; rows >= T are zero.
//
// stat_tiles: [H, Tpad / 128, 2] tiles of 4 KB for the dK/dV kernel, which adds the per-query-column terms to S^T and
// dP^T with one extra MMA step each instead of reading them in the softmax loop: D[i][j] += sum_k ONES[i][k] * C[j][k]
// with C[j][0..15] = {hi, lo, 0 x 6, hi, lo, 0 x 6}, hi + lo the bf16 split of HALF the term (both 16-byte halves are
// equal, so the operand does not depend on which half the hardware takes as k = 0..7).  Tile 0 carries -lse / scale
// (so that (S^T + c) * scale * log2 e = s * scale * log2 e - lse * log2 e), tile 1 carries -delta.  Layout: 8-row groups
// of 256 bytes; inside a group the first 16-byte halves of the 8 rows, then the second halves.
__global__ void prep_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                            const float* __restrict__ lse, float* __restrict__ delta_pad, float* __restrict__ lse2_pad,
                            uint8_t* __restrict__ stat_tiles, float inv_scale,
                            int T, int Tpad, int H, int64_t do_row, int64_t o_row) {
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= Tpad * H) return;
  const int t = warp_global / H, h = warp_global % H;
  float s = 0.f, l2 = 0.f, l1 = 0.f;
  if (t < T) {
    const uint2 a = *reinterpret_cast<const uint2*>(dO + (int64_t)t * do_row + h * HD + lane * 4);
    const uint2 b = *reinterpret_cast<const uint2*>(O + (int64_t)t * o_row + h * HD + lane * 4);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(b2[i]);
      s += x.x * y.x + x.y * y.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    l1 = lse[(int64_t)h * T + t];
    l2 = l1 * LOG2E;
  }
  if (lane == 0) {
    delta_pad[(int64_t)h * Tpad + t] = -s;
    lse2_pad[(int64_t)h * Tpad + t] = -l2;
    const int blk = t / BLK, row = t % BLK;
    uint8_t* tile = stat_tiles + ((int64_t)h * (Tpad / BLK) + blk) * STAT_BYTES + (row >> 3) * 256 + (row & 7) * 16;
    const float c[2] = {-0.5f * l1 * inv_scale, -0.5f * s};
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      const __nv_bfloat16 hi = __float2bfloat16_rn(c[w]);
      const __nv_bfloat16 lo = __float2bfloat16_rn(c[w] - __bfloat162float(hi));
      const uint4 v = make_uint4((uint32_t)__bfloat16_as_ushort(hi) | ((uint32_t)__bfloat16_as_ushort(lo) << 16), 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(tile + w * STAT_TILE) = v;
      *reinterpret_cast<uint4*>(tile + w * STAT_TILE + 128) = v;
    }
  }
}

// ------------------------------------------------------------------------------------------- dK / dV
struct BarsKV {
  uint64_t kv_full;
  uint64_t q_full[STAGES], q_empty[STAGES];      // Q block + its lse2 / delta rows
  uint64_t d_full[STAGES], d_empty[STAGES];      // dO block
  uint64_t s_full, dp_full, p_full, ds_full;     // one completion per block each: parity = block & 1
  uint64_t acc_done, drain;
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int KV_SMEM_TILES = 2 * BIG_BYTES + STAGES * (2 * BLK_BYTES + STAT_BYTES) + STAT_TILE;   // + the all-ones operand
constexpr int KV_SMEM_TOTAL = KV_SMEM_TILES + 256 + 1024;
// TMEM columns: S^T 0..127 (P^T, bf16, overwrites 0..63), dP^T 128..255 (dS^T overwrites 128..191), dV 256, dK 384
constexpr uint32_t COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 384;

// Optional redirection of an output: rows [d * rows, (d + 1) * rows) go to tensor map m[d] instead of the
// kernel's own output map (another rank's buffer: the Ulysses head->sequence exchange of the gradient).
struct SplitMaps {
  CUtensorMap m[8];
  int rows;     // 0 = unused
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                      const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV,
                      const uint8_t* __restrict__ stat_tiles, int Tq, int Tk, int Tq_pad,
                      int H, int Hkv, int causal, float scale, int* __restrict__ err, long long* __restrict__ dbg,
                      const __grid_constant__ SplitMaps dk_split, const __grid_constant__ SplitMaps dv_split) {
#ifndef ODY_ATTN_TRACE
  dbg = nullptr;   // the clock-stamp timeline is a development aid: compiled out of the product kernels
#endif
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + BIG_BYTES;
  uint8_t* sQs = smem + 2 * BIG_BYTES;                    // STAGES Q blocks
  uint8_t* sDs = sQs + STAGES * BLK_BYTES;                // STAGES dO blocks
  uint8_t* sStat = sDs + STAGES * BLK_BYTES;              // per stage: -lse/scale tile | -delta tile
  uint8_t* sOnes = sStat + STAGES * STAT_BYTES;           // 128 x 16 bf16 ones: the A operand of the statistics step
  BarsKV* bars = (BarsKV*)(smem + KV_SMEM_TILES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, kvh = blockIdx.y;
  const int kv0 = kt * BIG;
  const int G = H / Hkv;
  const int nq = (Tq + BLK - 1) / BLK;
  const int i0 = causal ? min(nq, kv0 / BLK) : 0;          // first query block that sees this KV tile
  const int per_head = nq - i0;
  const int total = per_head * G;

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->q_full[s], 1); mbar_init(&bars->q_empty[s], 1);
      mbar_init(&bars->d_full[s], 1); mbar_init(&bars->d_empty[s], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->p_full, 256);
    mbar_init(&bars->ds_full, 256);
    mbar_init(&bars->acc_done, 1);
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
  for (int i = threadIdx.x; i < STAT_TILE / 16; i += NUM_THREADS)
    reinterpret_cast<uint4*>(sOnes)[i] = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
  fence_proxy_async_smem();       // the tensor core reads sOnes through the async proxy
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp < 4) {
   reg_dec<REGS_ISSUE>();
   if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bars->kv_full, 2 * BIG_BYTES);
      tma_load_3d(sK, &tmK, 0, kvh, kv0, &bars->kv_full);
      tma_load_3d(sK + BIG_HALF, &tmK, 64, kvh, kv0, &bars->kv_full);
      tma_load_3d(sV, &tmV, 0, kvh, kv0, &bars->kv_full);
      tma_load_3d(sV + BIG_HALF, &tmV, 64, kvh, kv0, &bars->kv_full);
      for (int it = 0; it < total; ++it) {
        const int stage = it % STAGES;
        const uint32_t phase = (it / STAGES) & 1;
        const int head = kvh * G + it / per_head;
        const int qrow = (i0 + it % per_head) * BLK;
        // the Q ring is released by dK, the dO ring (earlier) by dV
        if (!mbar_wait(&bars->q_empty[stage], phase ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
        uint8_t* sQ = sQs + stage * BLK_BYTES;
        mbar_expect_tx(&bars->q_full[stage], BLK_BYTES + STAT_BYTES);
        tma_load_3d(sQ, &tmQ, 0, head, qrow, &bars->q_full[stage]);
        tma_load_3d(sQ + BLK_HALF, &tmQ, 64, head, qrow, &bars->q_full[stage]);
        bulk_load_1d(sStat + stage * STAT_BYTES, stat_tiles + ((int64_t)head * (Tq_pad / BLK) + qrow / BLK) * STAT_BYTES, STAT_BYTES,
                     &bars->q_full[stage]);
        if (!mbar_wait(&bars->d_empty[stage], phase ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
        uint8_t* sD = sDs + stage * BLK_BYTES;
        mbar_expect_tx(&bars->d_full[stage], BLK_BYTES);
        tma_load_3d(sD, &tmDO, 0, head, qrow, &bars->d_full[stage]);
        tma_load_3d(sD + BLK_HALF, &tmDO, 64, head, qrow, &bars->d_full[stage]);
      }
    }
  } else if (warp == 1) {
    {
      // every lane runs the control flow, so the compiler keeps descriptors and loop state in uniform registers;
      // one elected lane issues the tcgen05 instructions (see the note on the issue rate in flash_fwd.cu)
      const bool leader = elect_one();
      constexpr uint32_t IDESC_S = make_idesc_bf16(BIG, BLK, 0, 0);
      constexpr uint32_t IDESC_ACC = make_idesc_bf16(BIG, HD, 0, 1);
      bool ok = mbar_wait(&bars->kv_full, 0, abort_flag, err, ODY_ERR_TIMEOUT_FULL);
      const uint64_t kdesc0 = make_smem_desc(smem_u32(sK), 16, 1024), vdesc0 = make_smem_desc(smem_u32(sV), 16, 1024);
      const uint64_t q_k0 = make_smem_desc(smem_u32(sQs), 16, 1024), d_k0 = make_smem_desc(smem_u32(sDs), 16, 1024);
      const uint64_t q_mn0 = make_smem_desc(smem_u32(sQs), BLK_HALF, 1024), d_mn0 = make_smem_desc(smem_u32(sDs), BLK_HALF, 1024);
      const uint64_t ones_d = make_smem_desc_noswizzle(smem_u32(sOnes), 128, 256);
      const uint64_t stat_d0 = make_smem_desc_noswizzle(smem_u32(sStat), 128, 256);
      const bool trace = dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
      // S^T(it) = K Q^T - lse / scale (per query column): waits for the Q block
      auto issue_s = [&](int it) -> bool {
        const int stage = it % STAGES;
        if (!mbar_wait(&bars->q_full[stage], (it / STAGES) & 1, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint64_t qd = desc_advance(q_k0, stage * BLK_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * BIG_HALF + (kk & 3) * 32;
          if (leader) umma_ss(tmem + COL_ST, desc_advance(kdesc0, off), desc_advance(qd, off), IDESC_S, kk > 0 ? 1u : 0u);
        }
        if (leader) umma_ss(tmem + COL_ST, ones_d, desc_advance(stat_d0, stage * STAT_BYTES), IDESC_S, 1u);
        if (leader) umma_commit(&bars->s_full);
        return true;
      };
      // dP^T(it) = V dO^T: waits for the dO block
      auto issue_dp = [&](int it) -> bool {
        const int stage = it % STAGES;
        if (!mbar_wait(&bars->d_full[stage], (it / STAGES) & 1, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint64_t dd = desc_advance(d_k0, stage * BLK_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * BIG_HALF + (kk & 3) * 32;
          if (leader) umma_ss(tmem + COL_DPT, desc_advance(vdesc0, off), desc_advance(dd, off), IDESC_S, kk > 0 ? 1u : 0u);
        }
        // dP^T - delta: the statistics tile of this block came with its Q block, which S^T(it) already waited for
        if (leader) umma_ss(tmem + COL_DPT, ones_d, desc_advance(stat_d0, stage * STAT_BYTES + STAT_TILE), IDESC_S, 1u);
        if (leader) umma_commit(&bars->dp_full);
        return true;
      };
      if (ok && total > 0) ok = issue_s(0) && issue_dp(0);
      // One warp issues all four products of a block (every lane runs the loop, one elected lane issues: see the note in
      // flash_fwd.cu; 752 -> 797 and 879 -> 930 TFLOP/s for the two backward kernels together).  Measured before that and
      // not kept: two issuing warps on two schedulers (warp 1: dV(it), S^T(it+1); warp 2: dK(it), dP^T(it+1); the same
      // split in the dQ kernel): with two queues the pipe interleaves their instructions and every product completes
      // later, 688 / 800 TFLOP/s.
      // The tensor pipe executes in issue order, so S^T(it+1) may overwrite P^T(it) once dV(it) has been issued,
      // and dP^T(it+1) may overwrite dS^T(it) once dK(it) has.  While the softmax warps turn dP^T(it) into
      // dS^T(it) the pipe runs dV(it) and S^T(it+1); while they turn S^T(it+1) into P^T(it+1) it runs dK(it)
      // and dP^T(it+1).
      for (int it = 0; it < total && ok; ++it) {
        const int stage = it % STAGES;
        const uint32_t par = it & 1;
        const uint32_t acc0 = it > 0 ? 1u : 0u;
        if (trace && it < 48) dbg[it * 8 + 0] = clock64();
        if (!mbar_wait(&bars->p_full, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        if (trace && it < 48) dbg[it * 8 + 1] = clock64();                 // P^T(it) seen
        tc_fence_after();
        const uint64_t dmn = desc_advance(d_mn0, stage * BLK_BYTES);
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk)      // dV += P^T dO
          if (leader) umma_ts(tmem + COL_DV, tmem + COL_ST + kk * 8, desc_advance(dmn, kk * 2048), IDESC_ACC, kk > 0 ? 1u : acc0);
        if (leader) umma_commit(&bars->d_empty[stage]);
        if (it + 1 < total && !issue_s(it + 1)) { ok = false; break; }
        if (!mbar_wait(&bars->ds_full, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint64_t qmn = desc_advance(q_mn0, stage * BLK_BYTES);
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk)      // dK += dS^T Q
          if (leader) umma_ts(tmem + COL_DK, tmem + COL_DPT + kk * 8, desc_advance(qmn, kk * 2048), IDESC_ACC, kk > 0 ? 1u : acc0);
        if (leader) umma_commit(&bars->q_empty[stage]);
        if (it + 1 < total && !issue_dp(it + 1)) { ok = false; break; }
      }
      if (ok) {
        if (leader) umma_commit(&bars->acc_done);
      } else {
        if (leader) umma_commit(&bars->drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(&bars->drain, 0) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
      }
    }
   }
  } else {
    reg_inc<REGS_MATH>();
    const int q = warp & 3;                               // TMEM lane quarter
    const int hf = (warp - 4) >> 2;                       // which 64 of the block's 128 query columns this warp handles
    const int r = q * 32 + lane;                          // kv row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const float sl2 = scale * LOG2E;
    const uint64_t sl2_2 = pk2(sl2, sl2);
    bool ok = true;
    for (int it = 0; it < total; ++it) {
      const uint32_t par = it & 1;
      const int qrow0 = (i0 + it % per_head) * BLK + hf * 64;
      const bool strace = dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 128 && it < 48;
      // ---- part 1: S^T -> P^T
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL));
      if (strace) dbg[it * 8 + 2] = clock64();                             // S^T(it) complete
      uint32_t sv[64];
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32(tmem + COL_ST + hf * 64 + lane_off, sv);
        tmem_ld_32x32(tmem + COL_ST + hf * 64 + 32 + lane_off, sv + 32);
        tmem_ld_wait();
      }
      // P^T is written over the first 64 columns of S^T: the other warp of this lane quarter must have read
      // its inputs before either of us stores; the two also agree here on leaving the loop
      if (!named_barrier_and(4 + q, 64, ok)) { ok = false; break; }
      if (strace) dbg[it * 8 + 3] = clock64();                             // S^T in registers, pair agreed
      const bool diag = causal && (qrow0 < kv0 + BIG);     // some (q, kv) pairs of this half block are masked
      {
        uint32_t pp[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          // the accumulator already holds s - lse / scale: x = that * scale * log2(e), two query columns at once
          const uint64_t x2 = mul2(pk2u(sv[2 * c], sv[2 * c + 1]), sl2_2);
          float p0, p1;
          if ((c % ODY_BWD_POLY_DEN) < ODY_BWD_POLY_NUM) {
            exp2_poly2(x2, p0, p1);
          } else {
            upk2(x2, p0, p1);
            p0 = exp2_mufu(p0);
            p1 = exp2_mufu(p1);
          }
          if (diag) {
            if (qrow0 + 2 * c < kv0 + r) p0 = 0.f;
            if (qrow0 + 2 * c + 1 < kv0 + r) p1 = 0.f;
          }
          sv[2 * c] = __float_as_uint(p0);
          sv[2 * c + 1] = __float_as_uint(p1);
          pp[c] = pack_bf16(p0, p1);
        }
        if (dbg != nullptr) {   // tracing only: pin every packed value before the stamp
          asm volatile("" ::"r"(pp[0]), "r"(pp[1]), "r"(pp[2]), "r"(pp[3]), "r"(pp[4]), "r"(pp[5]), "r"(pp[6]), "r"(pp[7]), "r"(pp[8]), "r"(pp[9]), "r"(pp[10]), "r"(pp[11]), "r"(pp[12]), "r"(pp[13]), "r"(pp[14]), "r"(pp[15]));
          asm volatile("" ::"r"(pp[16]), "r"(pp[17]), "r"(pp[18]), "r"(pp[19]), "r"(pp[20]), "r"(pp[21]), "r"(pp[22]), "r"(pp[23]), "r"(pp[24]), "r"(pp[25]), "r"(pp[26]), "r"(pp[27]), "r"(pp[28]), "r"(pp[29]), "r"(pp[30]), "r"(pp[31]));
        }
        if (strace) dbg[it * 8 + 4] = clock64();                           // P^T computed
        tmem_st_32x16(tmem + COL_ST + hf * 32 + lane_off, pp);
        tmem_st_32x16(tmem + COL_ST + hf * 32 + 16 + lane_off, pp + 16);
        tmem_st_wait();
        if (strace) dbg[it * 8 + 5] = clock64();                           // P^T stored
        tc_fence_before();
        mbar_arrive(&bars->p_full);
      }
      // ---- part 2: dP^T -> dS^T = P^T * (dP^T - delta) * scale
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->dp_full, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL));
      uint32_t dp[64];
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32(tmem + COL_DPT + hf * 64 + lane_off, dp);
        tmem_ld_32x32(tmem + COL_DPT + hf * 64 + 32 + lane_off, dp + 32);
        tmem_ld_wait();
      }
      if (!named_barrier_and(4 + q, 64, ok)) { ok = false; break; }
      if (strace) dbg[it * 8 + 6] = clock64();                             // dP^T in registers, pair agreed
      {
        uint32_t ds[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          // dS = P * (dP - delta), the accumulator already holding dP - delta; the softmax scale is applied once, to
          // dK, in the epilogue
          float d0, d1;
          upk2(mul2(pk2u(sv[2 * c], sv[2 * c + 1]), pk2u(dp[2 * c], dp[2 * c + 1])), d0, d1);
          ds[c] = pack_bf16(d0, d1);
        }
        tmem_st_32x16(tmem + COL_DPT + hf * 32 + lane_off, ds);
        tmem_st_32x16(tmem + COL_DPT + hf * 32 + 16 + lane_off, ds + 16);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&bars->ds_full);
      }
      if (strace) dbg[it * 8 + 7] = clock64();
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_done, 0, abort_flag, err, ODY_ERR_TIMEOUT_MISC));
    if (ok) {
      tc_fence_after();
      // dV -> sV region, dK -> sK region (both dead now), bf16, swizzled for the TMA store; this warp converts
      // output columns [hf * 64, hf * 64 + 64), which is exactly one 64-column half of the staging tile
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        uint8_t* dst = (which == 0 ? sV : sK) + hf * BIG_HALF;
        const uint32_t col = (which == 0 ? COL_DV : COL_DK) + hf * 64;
        const float mult = which == 0 ? 1.f : scale;       // dK = scale * dS^T Q
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[16];
          tmem_ld_32x16(tmem + col + lane_off + c * 16, o);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 16; ++t) o[t] = __float_as_uint(__uint_as_float(o[t]) * mult);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            uint4 v4;
            v4.x = pack_bf16(__uint_as_float(o[8 * t + 0]), __uint_as_float(o[8 * t + 1]));
            v4.y = pack_bf16(__uint_as_float(o[8 * t + 2]), __uint_as_float(o[8 * t + 3]));
            v4.z = pack_bf16(__uint_as_float(o[8 * t + 4]), __uint_as_float(o[8 * t + 5]));
            v4.w = pack_bf16(__uint_as_float(o[8 * t + 6]), __uint_as_float(o[8 * t + 7]));
            const int chunk = c * 2 + t;
            *reinterpret_cast<uint4*>(dst + r * 128 + ((chunk ^ (r & 7)) << 4)) = v4;
          }
        }
      }
      fence_proxy_async_smem();
    }
    tc_fence_before();
    named_barrier(1, 256);
    if (ok && warp == 4 && lane == 0 && !*abort_flag) {
      const int d = dk_split.rows > 0 ? kv0 / dk_split.rows : 0;
      const int row = dk_split.rows > 0 ? kv0 - d * dk_split.rows : kv0;
      const CUtensorMap* mV = dk_split.rows > 0 ? &dv_split.m[d] : &tmDV;
      const CUtensorMap* mK = dk_split.rows > 0 ? &dk_split.m[d] : &tmDK;
      tma_store_3d(mV, sV, 0, kvh, row);
      tma_store_3d(mV, sV + BIG_HALF, 64, kvh, row);
      tma_store_3d(mK, sK, 0, kvh, row);
      tma_store_3d(mK, sK + BIG_HALF, 64, kvh, row);
      tma_store_commit();
      tma_store_wait<0>();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// ------------------------------------------------------------------------------------------- dK / dV / dQ in one kernel
// The split pair above computes S and dP twice (seven 128 x 128 x 128 products per (query block, KV tile) pair) to stay
// free of atomics.  This kernel computes them once (five products) and is the default: same grid and streaming as the
// dK/dV kernel, plus
//   * dS^T leaves the softmax warps through SHARED memory instead of TMEM ([128 kv rows][128 query columns] bf16, the
//     layout of a K tile): read K-major it is the A operand of dK += dS^T Q, read MN-major it is the A operand of
//     dQ_blk = dS K (K itself, resident, is the MN-major B operand);
//   * dQ_blk (this KV tile's contribution to one query block) accumulates in the TMEM columns of dP^T, which are free once
//     the softmax warps hold dP^T in registers; the same warps drain it (query rows on lanes) and add it to an fp32
//     [H, Tq_pad, 128] accumulator with vector reductions (red.global.add.v4.f32) - contributions of different KV tiles
//     arrive in no fixed order, so dQ is reproducible only up to fp32 summation order; a small kernel scales and rounds
//     it to bf16 afterwards (and performs the Ulysses row split);
//   * the dO ring has ONE stage (dO(i+1) is fetched while S^T(i+1), dQ(i) and dK(i) run) to make room for the dS^T tile.
// Issue order per block: dV(i), S^T(i+1), dQ(i), dK(i), dP^T(i+1); dK(i) runs while dQ(i) is drained.
struct BarsF {
  uint64_t kv_full;
  uint64_t q_full[STAGES], q_empty[STAGES];      // Q block + its statistics tiles
  uint64_t d_full, d_empty;                      // the single dO block
  uint64_t s_full, dp_full, p_full, ds_full;     // one completion per block each: parity = block & 1
  uint64_t dq_full, dq_free, ds_free;
  uint64_t acc_done, drain;
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int F_SMEM_TILES = 2 * BIG_BYTES + STAGES * (BLK_BYTES + STAT_BYTES) + BLK_BYTES + BLK_BYTES + STAT_TILE;
constexpr int F_SMEM_TOTAL = F_SMEM_TILES + 256 + 1024;
static_assert(F_SMEM_TOTAL <= 232448, "fused backward exceeds the shared memory of an SM");
// the issuing thread of this kernel juggles more descriptors than those of the split kernels
constexpr int F_REGS_ISSUE = 72, F_REGS_MATH = 216;
static_assert(128 * F_REGS_ISSUE + 256 * F_REGS_MATH <= NUM_THREADS * REGS_LAUNCH, "setmaxnreg split exceeds the CTA's registers");

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// (Staging dQ_blk in the dS^T tile and adding it with TMA reductions, cp.reduce.async.bulk.tensor, measured slower than
// the per-thread vector reductions: 2.32 ms against 2.02 ms at T = 8192 x 32 heads.  Either way the L2 absorbs the
// partial dQ at about 2.2 TB/s, which is what bounds this kernel.)
__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                       const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV,
                       const uint8_t* __restrict__ stat_tiles, float* __restrict__ dq_acc, int Tq, int Tk, int Tq_pad,
                       int H, int Hkv, int causal, float scale, int* __restrict__ err,
                       const __grid_constant__ SplitMaps dk_split, const __grid_constant__ SplitMaps dv_split) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + BIG_BYTES;
  uint8_t* sQs = smem + 2 * BIG_BYTES;                    // STAGES Q blocks
  uint8_t* sD = sQs + STAGES * BLK_BYTES;                 // the dO block
  uint8_t* sDS = sD + BLK_BYTES;                          // dS^T of the current block
  uint8_t* sStat = sDS + BLK_BYTES;                       // per Q stage: -lse/scale tile | -delta tile
  uint8_t* sOnes = sStat + STAGES * STAT_BYTES;           // 128 x 16 bf16 ones: the A operand of the statistics step
  BarsF* bars = (BarsF*)(smem + F_SMEM_TILES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, kvh = blockIdx.y;
  const int kv0 = kt * BIG;
  const int G = H / Hkv;
  const int nq = (Tq + BLK - 1) / BLK;
  const int i0 = causal ? min(nq, kv0 / BLK) : 0;          // first query block that sees this KV tile
  const int per_head = nq - i0;
  const int total = per_head * G;
  // (Starting each CTA's walk over the query blocks at a different block, so that concurrent CTAs add to different
  // lines of the dQ accumulator, measured no faster: the reductions are bound by volume, not by collisions.)
  auto q_block = [&](int it) { return i0 + it % per_head; };

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&bars->q_full[s], 1); mbar_init(&bars->q_empty[s], 1); }
    mbar_init(&bars->d_full, 1); mbar_init(&bars->d_empty, 1);
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->p_full, 256);
    mbar_init(&bars->ds_full, 256);
    mbar_init(&bars->dq_full, 1);
    mbar_init(&bars->dq_free, 256);
    mbar_init(&bars->ds_free, 1);
    mbar_init(&bars->acc_done, 1);
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
  for (int i = threadIdx.x; i < STAT_TILE / 16; i += NUM_THREADS)
    reinterpret_cast<uint4*>(sOnes)[i] = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
  fence_proxy_async_smem();       // the tensor core reads sOnes through the async proxy
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp < 4) {
   reg_dec<F_REGS_ISSUE>();
   if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bars->kv_full, 2 * BIG_BYTES);
      tma_load_3d(sK, &tmK, 0, kvh, kv0, &bars->kv_full);
      tma_load_3d(sK + BIG_HALF, &tmK, 64, kvh, kv0, &bars->kv_full);
      tma_load_3d(sV, &tmV, 0, kvh, kv0, &bars->kv_full);
      tma_load_3d(sV + BIG_HALF, &tmV, 64, kvh, kv0, &bars->kv_full);
      int issued_q = 0, issued_d = 0;
      for (int it = 0; it < total; ++it) {
        const int stage = it % STAGES;
        const uint32_t phase = (it / STAGES) & 1;
        const int head = kvh * G + it / per_head;
        const int qrow = q_block(it) * BLK;
        if (!mbar_wait(&bars->q_empty[stage], phase ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
        uint8_t* sQ = sQs + stage * BLK_BYTES;
        mbar_expect_tx(&bars->q_full[stage], BLK_BYTES + STAT_BYTES);
        tma_load_3d(sQ, &tmQ, 0, head, qrow, &bars->q_full[stage]);
        tma_load_3d(sQ + BLK_HALF, &tmQ, 64, head, qrow, &bars->q_full[stage]);
        bulk_load_1d(sStat + stage * STAT_BYTES, stat_tiles + ((int64_t)head * (Tq_pad / BLK) + qrow / BLK) * STAT_BYTES, STAT_BYTES,
                     &bars->q_full[stage]);
        ++issued_q;
        // the single dO slot is released by dV of the block before
        if (!mbar_wait(&bars->d_empty, (it & 1) ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&bars->d_full, BLK_BYTES);
        tma_load_3d(sD, &tmDO, 0, head, qrow, &bars->d_full);
        tma_load_3d(sD + BLK_HALF, &tmDO, 64, head, qrow, &bars->d_full);
        ++issued_d;
      }
      if (*abort_flag) {
        // somebody gave up: let the copies still in flight land before the CTA's shared memory goes away (bounded)
        const long long t0 = clock64();
        for (int b = 0; b < 2; ++b) {
          const int jq = issued_q - 1 - b;
          while (jq >= 0 && !mbar_try_wait(&bars->q_full[jq % STAGES], (jq / STAGES) & 1) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
        }
        const int jd = issued_d - 1;
        while (jd >= 0 && !mbar_try_wait(&bars->d_full, jd & 1) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
      }
    }
  } else if (warp == 1) {
    {
      // every lane runs the control flow, so the compiler keeps descriptors and loop state in uniform registers;
      // one elected lane issues the tcgen05 instructions (see the note on the issue rate in flash_fwd.cu)
      const bool leader = elect_one();
      constexpr uint32_t IDESC_S = make_idesc_bf16(BIG, BLK, 0, 0);      // S^T, dP^T: both operands K-major
      constexpr uint32_t IDESC_ACC = make_idesc_bf16(BIG, HD, 0, 1);     // dV (A in TMEM), dK (A K-major): B MN-major
      constexpr uint32_t IDESC_DQ = make_idesc_bf16(BLK, HD, 1, 1);      // dQ_blk: A = dS MN-major, B = K MN-major
      bool ok = mbar_wait(&bars->kv_full, 0, abort_flag, err, ODY_ERR_TIMEOUT_FULL);
      uint64_t kdesc0 = make_smem_desc(smem_u32(sK), 16, 1024), vdesc0 = make_smem_desc(smem_u32(sV), 16, 1024);
      uint64_t k_mn = make_smem_desc(smem_u32(sK), BIG_HALF, 1024);
      uint64_t q_k0 = make_smem_desc(smem_u32(sQs), 16, 1024), d_k = make_smem_desc(smem_u32(sD), 16, 1024);
      uint64_t q_mn0 = make_smem_desc(smem_u32(sQs), BLK_HALF, 1024), d_mn = make_smem_desc(smem_u32(sD), BLK_HALF, 1024);
      uint64_t ds_k = make_smem_desc(smem_u32(sDS), 16, 1024), ds_mn = make_smem_desc(smem_u32(sDS), BLK_HALF, 1024);
      const uint64_t ones_d = make_smem_desc_noswizzle(smem_u32(sOnes), 128, 256);
      const uint64_t stat_d0 = make_smem_desc_noswizzle(smem_u32(sStat), 128, 256);
      // Nine descriptor bases times eight slice offsets each are loop invariants the compiler would rather keep in
      // ~110 registers than recompute with one add per MMA; this thread has no such room.  Passing the bases through
      // an empty asm each iteration makes them opaque, so the sums are formed where they are used.
      auto opaque = [&]() {
        asm volatile("" : "+l"(kdesc0), "+l"(vdesc0), "+l"(k_mn), "+l"(q_k0), "+l"(d_k), "+l"(q_mn0), "+l"(d_mn), "+l"(ds_k), "+l"(ds_mn));
      };
      // S^T(it) = K Q^T - lse / scale (per query column): waits for the Q block
      auto issue_s = [&](int it) -> bool {
        const int stage = it % STAGES;
        if (!mbar_wait(&bars->q_full[stage], (it / STAGES) & 1, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint64_t qd = desc_advance(q_k0, stage * BLK_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * BIG_HALF + (kk & 3) * 32;
          if (leader) umma_ss(tmem + COL_ST, desc_advance(kdesc0, off), desc_advance(qd, off), IDESC_S, kk > 0 ? 1u : 0u);
        }
        if (leader) umma_ss(tmem + COL_ST, ones_d, desc_advance(stat_d0, stage * STAT_BYTES), IDESC_S, 1u);
        if (leader) umma_commit(&bars->s_full);
        return true;
      };
      // dP^T(it) = V dO^T - delta: waits for the dO block (its statistics tile came with the Q block)
      auto issue_dp = [&](int it) -> bool {
        const int stage = it % STAGES;
        if (!mbar_wait(&bars->d_full, it & 1, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * BIG_HALF + (kk & 3) * 32;
          if (leader) umma_ss(tmem + COL_DPT, desc_advance(vdesc0, off), desc_advance(d_k, off), IDESC_S, kk > 0 ? 1u : 0u);
        }
        if (leader) umma_ss(tmem + COL_DPT, ones_d, desc_advance(stat_d0, stage * STAT_BYTES + STAT_TILE), IDESC_S, 1u);
        if (leader) umma_commit(&bars->dp_full);
        return true;
      };
      if (ok && total > 0) ok = issue_s(0) && issue_dp(0);
      for (int it = 0; it < total && ok; ++it) {
        const int stage = it % STAGES;
        const uint32_t par = it & 1;
        const uint32_t acc0 = it > 0 ? 1u : 0u;
        opaque();
        if (!mbar_wait(&bars->p_full, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk)      // dV += P^T dO
          if (leader) umma_ts(tmem + COL_DV, tmem + COL_ST + kk * 8, desc_advance(d_mn, kk * 2048), IDESC_ACC, kk > 0 ? 1u : acc0);
        if (leader) umma_commit(&bars->d_empty);               // dO(it) is free: the producer fetches dO(it+1)
        if (it + 1 < total && !issue_s(it + 1)) { ok = false; break; }
        if (!mbar_wait(&bars->ds_full, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BIG / 16; ++kk)      // dQ_blk = dS K   (k runs over the 128 kv rows)
          if (leader) umma_ss(tmem + COL_DPT, desc_advance(ds_mn, kk * 2048), desc_advance(k_mn, kk * 2048), IDESC_DQ, kk > 0 ? 1u : 0u);
        if (leader) umma_commit(&bars->dq_full);
        const uint64_t qmn = desc_advance(q_mn0, stage * BLK_BYTES);
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk) {    // dK += dS^T Q   (k runs over the 128 query rows)
          const uint32_t off = (kk >> 2) * BLK_HALF + (kk & 3) * 32;
          if (leader) umma_ss(tmem + COL_DK, desc_advance(ds_k, off), desc_advance(qmn, kk * 2048), IDESC_ACC, kk > 0 ? 1u : acc0);
        }
        if (leader) umma_commit(&bars->q_empty[stage]);
        if (leader) umma_commit(&bars->ds_free);               // the dS^T tile may be overwritten
        if (it + 1 < total) {
          // dP^T(it+1) lands where dQ_blk(it) sits: the softmax warps must have drained it
          if (!mbar_wait(&bars->dq_free, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          if (!issue_dp(it + 1)) { ok = false; break; }
        }
      }
      if (ok) {
        if (leader) umma_commit(&bars->acc_done);
      } else {
        if (leader) umma_commit(&bars->drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(&bars->drain, 0) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
      }
    }
   }
  } else {
    reg_inc<F_REGS_MATH>();
    const int q = warp & 3;                               // TMEM lane quarter
    const int hf = (warp - 4) >> 2;                       // which 64 of 128 columns this warp handles
    const int r = q * 32 + lane;                          // TMEM lane: kv row for S^T / dP^T, query row for dQ_blk
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const float sl2 = scale * LOG2E;
    const uint64_t sl2_2 = pk2(sl2, sl2);
    bool ok = true;
    // dQ_blk(it) -> fp32 accumulator; this thread: query row r of the block, head-dim columns [hf * 64, hf * 64 + 64)
    auto drain_dq = [&](int it) -> bool {
      if (!ok) return false;
      bool good = __all_sync(0xffffffffu, mbar_wait(&bars->dq_full, it & 1, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL));
      if (!good) return false;
      tc_fence_after();
      const int head = kvh * G + it / per_head;
      const int qrow = q_block(it) * BLK + r;              // < Tq_pad: the accumulator has padded rows
      const int li = lane & 7;
      // Each thread gets 32 consecutive floats (one 128-byte line) of its own row per pass.  An 8 x 8 transpose of the
      // 16-byte chunks inside every group of 8 lanes (three butterfly steps of shuffles) makes step c of the write-out
      // cover the whole line of row 8 * group + c from 8 neighbouring lanes: full lines instead of 32 scattered pieces.
      auto transpose8 = [&](uint32_t* a) {
#pragma unroll
        for (int sft = 1; sft < 8; sft <<= 1) {
          const bool upper = (li & sft) != 0;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            if (c & sft) continue;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              const uint32_t send = upper ? a[4 * c + w] : a[4 * (c ^ sft) + w];
              const uint32_t got = __shfl_xor_sync(0xffffffffu, send, sft);
              if (upper) a[4 * c + w] = got; else a[4 * (c ^ sft) + w] = got;
            }
          }
        }
      };
      {
        float* dst = dq_acc + ((int64_t)head * Tq_pad + qrow) * HD + hf * 64;
        // two passes of 32 columns: the P values of part 1 stay in registers across this call
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t a[32];
          tmem_ld_32x32(tmem + COL_DPT + hf * 64 + half * 32 + lane_off, a);
          tmem_ld_wait();
          if (half == 1) {
            tc_fence_before();
            mbar_arrive(&bars->dq_free);                   // dQ_blk is out of TMEM: dP^T of the next block may land there
          }
          transpose8(a);
          float* line0 = dst - (int64_t)li * HD + half * 32 + 4 * li;     // row 8 * group, this lane's 16-byte chunk of it
#pragma unroll
          for (int c = 0; c < 8; ++c)
            red_add_v4(line0 + (int64_t)c * HD, __uint_as_float(a[4 * c]), __uint_as_float(a[4 * c + 1]),
                       __uint_as_float(a[4 * c + 2]), __uint_as_float(a[4 * c + 3]));
        }
      }
      return true;
    };
    // `ok` is warp-uniform.  The loop is left only at the pair barrier of part 1, where the two warps of a lane quarter
    // agree on it: a warp that has seen a wait give up skips the rest of its iteration and says so there.
    for (int it = 0; it < total; ++it) {
      const uint32_t par = it & 1;
      const int qrow0 = q_block(it) * BLK + hf * 64;
      // ---- part 1: S^T -> P^T (TMEM)
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL));
      uint32_t sv[64];
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32(tmem + COL_ST + hf * 64 + lane_off, sv);
        tmem_ld_32x32(tmem + COL_ST + hf * 64 + 32 + lane_off, sv + 32);
        tmem_ld_wait();
      }
      // P^T is written over the first 64 columns of S^T: the other warp of this lane quarter must have read
      // its inputs before either of us stores
      if (!named_barrier_and(4 + q, 64, ok)) { ok = false; break; }
      const bool diag = causal && (qrow0 < kv0 + BIG);     // some (q, kv) pairs of this half block are masked
      {
        uint32_t pp[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const uint64_t x2 = mul2(pk2u(sv[2 * c], sv[2 * c + 1]), sl2_2);
          float p0, p1;
          upk2(x2, p0, p1);
          p0 = exp2_mufu(p0);
          p1 = exp2_mufu(p1);
          if (diag) {
            if (qrow0 + 2 * c < kv0 + r) p0 = 0.f;
            if (qrow0 + 2 * c + 1 < kv0 + r) p1 = 0.f;
          }
          sv[2 * c] = __float_as_uint(p0);
          sv[2 * c + 1] = __float_as_uint(p1);
          pp[c] = pack_bf16(p0, p1);
        }
        tmem_st_32x16(tmem + COL_ST + hf * 32 + lane_off, pp);
        tmem_st_32x16(tmem + COL_ST + hf * 32 + 16 + lane_off, pp + 16);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&bars->p_full);
      }
      // ---- dQ_blk of the block before: its MMAs ran while part 1 was computed
      if (it > 0) ok = drain_dq(it - 1);
      // ---- part 2: dP^T -> dS^T = P^T * (dP^T - delta) -> shared memory
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->dp_full, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL));
      uint32_t dp[64];
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32(tmem + COL_DPT + hf * 64 + lane_off, dp);
        tmem_ld_32x32(tmem + COL_DPT + hf * 64 + 32 + lane_off, dp + 32);
        tmem_ld_wait();
      }
      // the tile still holds dS^T of the block before until dQ and dK of that block have read it
      if (ok && it > 0) ok = __all_sync(0xffffffffu, mbar_wait(&bars->ds_free, (it - 1) & 1, abort_flag, err, ODY_ERR_TIMEOUT_MISC));
      if (ok) {
        uint8_t* row = sDS + hf * BLK_HALF + r * 128;      // kv row r, query columns [hf * 64, hf * 64 + 64): one swizzled 128-byte row
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const int c = g * 4 + t;
            float d0, d1;
            upk2(mul2(pk2u(sv[2 * c], sv[2 * c + 1]), pk2u(dp[2 * c], dp[2 * c + 1])), d0, d1);
            w[t] = pack_bf16(d0, d1);
          }
          *reinterpret_cast<uint4*>(row + ((g ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        fence_proxy_async_smem();                           // the tensor core reads the tile through the async proxy
        tc_fence_before();                                  // and dP^T is in registers: its columns may take dQ_blk
        mbar_arrive(&bars->ds_full);
      }
    }
    if (ok && total > 0) ok = drain_dq(total - 1);
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_done, 0, abort_flag, err, ODY_ERR_TIMEOUT_MISC));
    if (ok) {
      tc_fence_after();
      // dV -> sV region, dK -> sK region (both dead now), bf16, swizzled for the TMA store
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        uint8_t* dst = (which == 0 ? sV : sK) + hf * BIG_HALF;
        const uint32_t col = (which == 0 ? COL_DV : COL_DK) + hf * 64;
        const float mult = which == 0 ? 1.f : scale;       // dK = scale * dS^T Q
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[16];
          tmem_ld_32x16(tmem + col + lane_off + c * 16, o);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 16; ++t) o[t] = __float_as_uint(__uint_as_float(o[t]) * mult);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            uint4 v4;
            v4.x = pack_bf16(__uint_as_float(o[8 * t + 0]), __uint_as_float(o[8 * t + 1]));
            v4.y = pack_bf16(__uint_as_float(o[8 * t + 2]), __uint_as_float(o[8 * t + 3]));
            v4.z = pack_bf16(__uint_as_float(o[8 * t + 4]), __uint_as_float(o[8 * t + 5]));
            v4.w = pack_bf16(__uint_as_float(o[8 * t + 6]), __uint_as_float(o[8 * t + 7]));
            const int chunk = c * 2 + t;
            *reinterpret_cast<uint4*>(dst + r * 128 + ((chunk ^ (r & 7)) << 4)) = v4;
          }
        }
      }
      fence_proxy_async_smem();
    }
    tc_fence_before();
    named_barrier(1, 256);
    if (ok && warp == 4 && lane == 0 && !*abort_flag) {
      const int d = dk_split.rows > 0 ? kv0 / dk_split.rows : 0;
      const int row = dk_split.rows > 0 ? kv0 - d * dk_split.rows : kv0;
      const CUtensorMap* mV = dk_split.rows > 0 ? &dv_split.m[d] : &tmDV;
      const CUtensorMap* mK = dk_split.rows > 0 ? &dk_split.m[d] : &tmDK;
      tma_store_3d(mV, sV, 0, kvh, row);
      tma_store_3d(mV, sV + BIG_HALF, 64, kvh, row);
      tma_store_3d(mK, sK, 0, kvh, row);
      tma_store_3d(mK, sK + BIG_HALF, 64, kvh, row);
      tma_store_commit();
      tma_store_wait<0>();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// dq [Tq, H, 128] bf16 (row pitch dq_row) = scale * acc [H, Tq_pad, 128]; with split_rows > 0 the rows go, in groups of
// split_rows, to dq_split.p[d] instead (possibly peer memory: plain 16-byte stores).
struct DqDests { __nv_bfloat16* p[8]; };
__global__ void dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, const __grid_constant__ DqDests split,
                                  int split_rows, int64_t dq_row, int Tq, int Tq_pad, int H, float scale) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;      // one thread per 8 elements
  const int64_t total = (int64_t)Tq * H * (HD / 8);
  if (idx >= total) return;
  const int c8 = (int)(idx % (HD / 8));
  const int h = (int)((idx / (HD / 8)) % H);
  const int t = (int)(idx / ((int64_t)(HD / 8) * H));
  const float* src = acc + ((int64_t)h * Tq_pad + t) * HD + c8 * 8;
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  uint4 o;
  o.x = pack_bf16(a.x * scale, a.y * scale);
  o.y = pack_bf16(a.z * scale, a.w * scale);
  o.z = pack_bf16(b.x * scale, b.y * scale);
  o.w = pack_bf16(b.z * scale, b.w * scale);
  __nv_bfloat16* base = dq;
  int row = t;
  if (split_rows > 0) {
    const int d = t / split_rows;
    base = split.p[d];
    row = t - d * split_rows;
  }
  *reinterpret_cast<uint4*>(base + (int64_t)row * dq_row + h * HD + c8 * 8) = o;
}

// ------------------------------------------------------------------------------------------- dQ
// Q and dO of the tile are the A operands of every S = Q K^T and dP = dO V^T of the kernel, so they live in TMEM (bf16,
// 64 columns each, written once by the softmax warps straight from global memory) and all 24 MMAs of a block are of the
// TS kind: only the streamed K / V block is read from shared memory, which is what bounds the rate of SS instructions.
constexpr int K_STAGES = 3;
struct BarsQ {
  uint64_t k_full[K_STAGES], k_empty[K_STAGES];
  uint64_t v_full[K_STAGES], v_empty[K_STAGES];
  uint64_t a_ready;                              // Q and dO are in TMEM
  uint64_t s_full, s_free, dp_full, ds_full;     // one completion per block each: parity = block & 1
  uint64_t acc_done, drain;
  uint32_t tmem_base;
  int abort_flag;
};
// A K block serves S(i) early and dQ(i) late, so its slot is held for a whole iteration and a half: with two slots the
// load of K(i+1) could only start when dQ(i-1) had finished and the MMA thread waited ~700 cycles per block for it.
constexpr int Q_SMEM_TILES = BIG_BYTES + 2 * K_STAGES * BLK_BYTES;       // dQ staging + K ring + V ring
constexpr int Q_SMEM_TOTAL = Q_SMEM_TILES + 256 + 1024;
// TMEM columns: S 0..127, dP 128..255 (dS, bf16, overwrites its first 64 columns), dQ 256..383, Q 384..447, dO 448..511
constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DQ = 256, COL_QA = 384, COL_DOA = 448;

__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_bwd_dq_kernel(const __nv_bfloat16* __restrict__ qg, const __nv_bfloat16* __restrict__ dog, int64_t q_row, int64_t do_row,
                    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const __grid_constant__ CUtensorMap tmDQ, const float* __restrict__ lse2_pad,
                    const float* __restrict__ delta_pad, int Tq, int Tk, int Tq_pad, int H, int Hkv, int causal,
                    float scale, int* __restrict__ err, const __grid_constant__ SplitMaps dq_split, long long* __restrict__ dbg) {
#ifndef ODY_ATTN_TRACE
  dbg = nullptr;   // the clock-stamp timeline is a development aid: compiled out of the product kernels
#endif
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                                     // staging of the dQ tile for its TMA store
  uint8_t* sKs = smem + BIG_BYTES;                        // K_STAGES K blocks
  uint8_t* sVs = sKs + K_STAGES * BLK_BYTES;              // K_STAGES V blocks
  BarsQ* bars = (BarsQ*)(smem + Q_SMEM_TILES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_q_tiles = (Tq + BIG - 1) / BIG;
  const int qt = causal ? (num_q_tiles - 1 - (int)blockIdx.x) : (int)blockIdx.x;
  const int head = blockIdx.y, kvh = head / (H / Hkv);
  const int q0 = qt * BIG;
  const int nk = (Tk + BLK - 1) / BLK;
  const int total = causal ? min(nk, (q0 + BIG) / BLK) : nk;

  if (threadIdx.x == 0) {
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(&bars->k_full[s], 1); mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1); mbar_init(&bars->v_empty[s], 1);
    }
    mbar_init(&bars->a_ready, 256);
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->s_free, 256);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->ds_full, 256);
    mbar_init(&bars->acc_done, 1);
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp < 4) {
   reg_dec<REGS_ISSUE>();
   if (warp == 0) {
    if (lane == 0) {
      for (int it = 0; it < total; ++it) {
        const int stage = it % K_STAGES;
        const uint32_t phase = (it / K_STAGES) & 1;
        if (!mbar_wait(&bars->k_empty[stage], phase ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
        uint8_t* sK = sKs + stage * BLK_BYTES;
        mbar_expect_tx(&bars->k_full[stage], BLK_BYTES);
        tma_load_3d(sK, &tmK, 0, kvh, it * BLK, &bars->k_full[stage]);
        tma_load_3d(sK + BLK_HALF, &tmK, 64, kvh, it * BLK, &bars->k_full[stage]);
        if (!mbar_wait(&bars->v_empty[stage], phase ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
        uint8_t* sV = sVs + stage * BLK_BYTES;
        mbar_expect_tx(&bars->v_full[stage], BLK_BYTES);
        tma_load_3d(sV, &tmV, 0, kvh, it * BLK, &bars->v_full[stage]);
        tma_load_3d(sV + BLK_HALF, &tmV, 64, kvh, it * BLK, &bars->v_full[stage]);
      }
    }
   } else if (warp == 1) {
    {
      // every lane runs the control flow, so the compiler keeps descriptors and loop state in uniform registers;
      // one elected lane issues the tcgen05 instructions (see the note on the issue rate in flash_fwd.cu)
      const bool leader = elect_one();
      constexpr uint32_t IDESC_S = make_idesc_bf16(BIG, BLK, 0, 0);
      constexpr uint32_t IDESC_ACC = make_idesc_bf16(BIG, HD, 0, 1);
      bool ok = mbar_wait(&bars->a_ready, 0, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL);
      tc_fence_after();
      const uint64_t k_k0 = make_smem_desc(smem_u32(sKs), 16, 1024), v_k0 = make_smem_desc(smem_u32(sVs), 16, 1024);
      const uint64_t k_mn0 = make_smem_desc(smem_u32(sKs), BLK_HALF, 1024);
      const bool trace = dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
      // S(it) = Q K^T, Q from TMEM
      auto issue_s = [&](int it) -> bool {
        const int stage = it % K_STAGES;
        if (!mbar_wait(&bars->k_full[stage], (it / K_STAGES) & 1, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint64_t kd = desc_advance(k_k0, stage * BLK_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          if (leader) umma_ts(tmem + COL_S, tmem + COL_QA + kk * 8, desc_advance(kd, (kk >> 2) * BLK_HALF + (kk & 3) * 32), IDESC_S, kk > 0 ? 1u : 0u);
        if (leader) umma_commit(&bars->s_full);
        return true;
      };
      // dP(it) = dO V^T, dO from TMEM
      auto issue_dp = [&](int it) -> bool {
        const int stage = it % K_STAGES;
        if (!mbar_wait(&bars->v_full[stage], (it / K_STAGES) & 1, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint64_t vd = desc_advance(v_k0, stage * BLK_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          if (leader) umma_ts(tmem + COL_DP, tmem + COL_DOA + kk * 8, desc_advance(vd, (kk >> 2) * BLK_HALF + (kk & 3) * 32), IDESC_S, kk > 0 ? 1u : 0u);
        if (leader) umma_commit(&bars->v_empty[stage]);
        if (leader) umma_commit(&bars->dp_full);
        return true;
      };
      if (ok && total > 0) ok = issue_s(0) && issue_dp(0);
      for (int it = 0; it < total && ok; ++it) {
        const uint32_t par = it & 1;
        if (trace && it < 48) dbg[it * 8 + 0] = clock64();                 // loop start
        if (it + 1 < total) {
          // S(it+1) overwrites S(it): the softmax warps must hold S(it) in registers
          if (!mbar_wait(&bars->s_free, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          if (trace && it < 48) dbg[it * 8 + 1] = clock64();               // S(it) freed
          if (!issue_s(it + 1)) { ok = false; break; }
          if (trace && it < 48) dbg[it * 8 + 2] = clock64();               // S(it+1) issued
        }
        if (!mbar_wait(&bars->ds_full, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        if (trace && it < 48) dbg[it * 8 + 3] = clock64();                 // dS(it) seen
        tc_fence_after();
        const uint64_t kmn = desc_advance(k_mn0, (it % K_STAGES) * BLK_BYTES);
        const uint32_t acc0 = it > 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk)   // dQ += dS K
          if (leader) umma_ts(tmem + COL_DQ, tmem + COL_DP + kk * 8, desc_advance(kmn, kk * 2048), IDESC_ACC, kk > 0 ? 1u : acc0);
        if (leader) umma_commit(&bars->k_empty[it % K_STAGES]);
        // dP(it+1) overwrites dS(it), which the in-order pipe has consumed with dQ(it) by then
        if (it + 1 < total && !issue_dp(it + 1)) { ok = false; break; }
      }
      if (ok) {
        if (leader) umma_commit(&bars->acc_done);
      } else {
        if (leader) umma_commit(&bars->drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(&bars->drain, 0) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
      }
    }
   }
  } else {
    reg_inc<REGS_MATH>();
    const int q = warp & 3;
    const int hf = (warp - 4) >> 2;                       // which 64 of the block's 128 key columns this warp handles
    const int r = q * 32 + lane;                          // query row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const float sl2 = scale * LOG2E;
    {
      // Q and dO rows of this thread, columns [hf * 64, hf * 64 + 64), into TMEM as bf16 pairs (rows past Tq are zero)
      const bool live = q0 + r < Tq;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const __nv_bfloat16* src = (which == 0 ? qg + (int64_t)(q0 + r) * q_row : dog + (int64_t)(q0 + r) * do_row) + head * HD + hf * 64;
        uint32_t a[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 v4 = live ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0u, 0u, 0u, 0u);
          a[4 * c] = v4.x; a[4 * c + 1] = v4.y; a[4 * c + 2] = v4.z; a[4 * c + 3] = v4.w;
        }
        tmem_st_32x32(tmem + (which == 0 ? COL_QA : COL_DOA) + hf * 32 + lane_off, a);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->a_ready);
    }
    const int64_t srow = (int64_t)head * Tq_pad + q0 + r;  // Tq_pad is a multiple of 128: every tile row has an entry
    const float nlse2 = lse2_pad[srow], ndelta = delta_pad[srow];      // stored negated
    const uint64_t sl2_2 = pk2(sl2, sl2), nlse2_2 = pk2(nlse2, nlse2), ndelta_2 = pk2(ndelta, ndelta);
    bool ok = true;
    for (int it = 0; it < total; ++it) {
      const uint32_t par = it & 1;
      const int kvb0 = it * BLK + hf * 64;
      const bool strace = dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 128 && it < 48;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL));
      if (strace) dbg[it * 8 + 4] = clock64();                             // S(it) complete
      uint32_t sv[64];
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32(tmem + COL_S + hf * 64 + lane_off, sv);
        tmem_ld_32x32(tmem + COL_S + hf * 64 + 32 + lane_off, sv + 32);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&bars->s_free);                       // S(it) is in registers
      }
      const bool diag = causal && (kvb0 + 63 > q0);
      const bool tail = kvb0 + 64 > Tk;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float p0, p1;
        upk2(fma2(pk2u(sv[2 * c], sv[2 * c + 1]), sl2_2, nlse2_2), p0, p1);
        p0 = exp2_mufu(p0);
        p1 = exp2_mufu(p1);
        if (diag) {
          if (kvb0 + 2 * c > q0 + r) p0 = 0.f;
          if (kvb0 + 2 * c + 1 > q0 + r) p1 = 0.f;
        }
        if (tail) {
          if (kvb0 + 2 * c >= Tk) p0 = 0.f;
          if (kvb0 + 2 * c + 1 >= Tk) p1 = 0.f;
        }
        sv[2 * c] = __float_as_uint(p0);
        sv[2 * c + 1] = __float_as_uint(p1);
      }
      if (strace) dbg[it * 8 + 5] = clock64();                             // P computed (as far as the compiler kept it here)
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->dp_full, par, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL));
      if (strace) dbg[it * 8 + 6] = clock64();                             // dP(it) complete
      uint32_t dp[64];
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32(tmem + COL_DP + hf * 64 + lane_off, dp);
        tmem_ld_32x32(tmem + COL_DP + hf * 64 + 32 + lane_off, dp + 32);
        tmem_ld_wait();
      }
      // dS overwrites dP's first 64 columns: both warps of the quarter have loaded; they also agree on leaving
      if (!named_barrier_and(4 + q, 64, ok)) { ok = false; break; }
      uint32_t ds[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        // dS = P * (dP - delta); the softmax scale is applied once, to dQ, in the epilogue
        float d0, d1;
        upk2(mul2(pk2u(sv[2 * c], sv[2 * c + 1]), add2(pk2u(dp[2 * c], dp[2 * c + 1]), ndelta_2)), d0, d1);
        ds[c] = pack_bf16(d0, d1);
      }
      tmem_st_32x16(tmem + COL_DP + hf * 32 + lane_off, ds);
      tmem_st_32x16(tmem + COL_DP + hf * 32 + 16 + lane_off, ds + 16);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->ds_full);
      if (strace) dbg[it * 8 + 7] = clock64();                             // dS published
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_done, 0, abort_flag, err, ODY_ERR_TIMEOUT_MISC));
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[16];
        tmem_ld_32x16(tmem + COL_DQ + hf * 64 + lane_off + c * 16, o);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          uint4 v4;
          v4.x = pack_bf16(__uint_as_float(o[8 * t + 0]) * scale, __uint_as_float(o[8 * t + 1]) * scale);
          v4.y = pack_bf16(__uint_as_float(o[8 * t + 2]) * scale, __uint_as_float(o[8 * t + 3]) * scale);
          v4.z = pack_bf16(__uint_as_float(o[8 * t + 4]) * scale, __uint_as_float(o[8 * t + 5]) * scale);
          v4.w = pack_bf16(__uint_as_float(o[8 * t + 6]) * scale, __uint_as_float(o[8 * t + 7]) * scale);
          const int chunk = c * 2 + t;
          *reinterpret_cast<uint4*>(sQ + hf * BIG_HALF + r * 128 + ((chunk ^ (r & 7)) << 4)) = v4;
        }
      }
      fence_proxy_async_smem();
    }
    tc_fence_before();
    named_barrier(1, 256);
    if (ok && warp == 4 && lane == 0 && !*abort_flag) {
      const int d = dq_split.rows > 0 ? q0 / dq_split.rows : 0;
      const int row = dq_split.rows > 0 ? q0 - d * dq_split.rows : q0;
      const CUtensorMap* mQ = dq_split.rows > 0 ? &dq_split.m[d] : &tmDQ;
      tma_store_3d(mQ, sQ, 0, head, row);
      tma_store_3d(mQ, sQ + BIG_HALF, 64, head, row);
      tma_store_commit();
      tma_store_wait<0>();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

}  // namespace bwd
}  // namespace ody

static long long* g_bwd_trace = nullptr;
// Optional per-block timelines (dK/dV kernel in the first 48 x 8 stamps, dQ kernel in the next 48 x 8)
// Optional per-block timeline of CTA (0,0) of the dK/dV kernel: 48 x 8 SM-clock stamps (see the kernel).
extern "C" void ody_flash_bwd_set_trace(long long* buf) { g_bwd_trace = buf; }

static int g_bwd_variant = 1;
// 1 (default): the split pair (dK/dV kernel + dQ kernel: seven products per block pair, no atomics, bitwise
// reproducible); 0: the fused dK/dV/dQ kernel (five products; dQ summed over KV tiles with fp32 reductions in no fixed
// order - at present the reduction traffic, not the tensor core, bounds it, and the split pair is the faster one)
extern "C" int ody_flash_bwd_set_variant(int v) {
  if (v < 0 || v > 1) return (int)cudaErrorInvalidValue;
  g_bwd_variant = v;
  return 0;
}

extern "C" int64_t ody_flash_bwd_workspace_bytes(int Tq, int H) {
  const int64_t Tpad = ((int64_t)Tq + 127) / 128 * 128;
  // -delta and exp2-domain -lse (padded), the statistics tiles, and the fp32 dQ accumulator of the fused kernel
  return 2 * (int64_t)H * Tpad * 4 + (int64_t)H * (Tpad / 128) * ody::bwd::STAT_BYTES + (int64_t)H * Tpad * ody::bwd::HD * 4;
}

// workspace: ody_flash_bwd_workspace_bytes(Tq, H) bytes, 16-byte aligned (delta and exp2-domain LSE, padded).
extern "C" int ody_flash_bwd(const void* dO, const void* q, const void* k, const void* v, const void* o, const float* lse,
                             void* dq, void* dk, void* dv, void* workspace, int Tq, int Tk, int H, int Hkv, int64_t do_row,
                             int64_t q_row, int64_t k_row, int64_t v_row, int64_t o_row, int64_t dq_row, int64_t dk_row,
                             int64_t dv_row, int causal, float scale, int* err, cudaStream_t st) {
  return ody_flash_bwd_ex(dO, q, k, v, o, lse, dq, dk, dv, workspace, Tq, Tk, H, Hkv, do_row, q_row, k_row, v_row, o_row, dq_row,
                          dk_row, dv_row, causal, scale, nullptr, nullptr, nullptr, 0, 0, err, st);
}

// Full form.  With n_split > 0 the gradients are not written to dq/dk/dv (which may then be null) but split by
// rows: rows [d * split_rows, (d + 1) * split_rows) of dq go to dq_split[d] ([split_rows, H, 128]), of dk / dv to
// dk_split[d] / dv_split[d] ([split_rows, Hkv, 128]); all with row pitches dq_row / dk_row / dv_row and possibly in
// peer memory.  split_rows % 128 == 0 and Tq == Tk.
extern "C" int ody_flash_bwd_ex(const void* dO, const void* q, const void* k, const void* v, const void* o, const float* lse,
                                void* dq, void* dk, void* dv, void* workspace, int Tq, int Tk, int H, int Hkv, int64_t do_row,
                                int64_t q_row, int64_t k_row, int64_t v_row, int64_t o_row, int64_t dq_row, int64_t dk_row,
                                int64_t dv_row, int causal, float scale, void* const* dq_split, void* const* dk_split,
                                void* const* dv_split, int n_split, int split_rows, int* err, cudaStream_t st) {
  using namespace ody;
  using namespace ody::bwd;
  SplitMaps sq, sk, sv;
  memset(&sq, 0, sizeof(sq));
  memset(&sk, 0, sizeof(sk));
  memset(&sv, 0, sizeof(sv));
  if (n_split > 0) {
    if (n_split > 8 || split_rows <= 0 || (split_rows % BIG) || Tq != Tk || (int64_t)split_rows * n_split < Tq) return (int)cudaErrorInvalidValue;
    if ((dq_row | dk_row | dv_row) % 8) return (int)cudaErrorInvalidValue;
    for (int d = 0; d < n_split; ++d) {
      if (((uintptr_t)dq_split[d] | (uintptr_t)dk_split[d] | (uintptr_t)dv_split[d]) & 15) return (int)cudaErrorInvalidValue;
      int e;
      if ((e = make_tmap_3d_bf16(&sq.m[d], dq_split[d], HD, H, split_rows, HD * 2, dq_row * 2, 64, 1, BIG))) return 795000 + e;
      if ((e = make_tmap_3d_bf16(&sk.m[d], dk_split[d], HD, Hkv, split_rows, HD * 2, dk_row * 2, 64, 1, BIG))) return 795000 + e;
      if ((e = make_tmap_3d_bf16(&sv.m[d], dv_split[d], HD, Hkv, split_rows, HD * 2, dv_row * 2, 64, 1, BIG))) return 795000 + e;
    }
    sq.rows = sk.rows = sv.rows = split_rows;
    // the unsplit maps below still need a valid address
    dq = dq_split[0]; dk = dk_split[0]; dv = dv_split[0];
  }
  if (Tq <= 0 || Tk <= 0 || H <= 0 || Hkv <= 0 || H % Hkv) return (int)cudaErrorInvalidValue;
  if (causal && Tq != Tk) return (int)cudaErrorInvalidValue;
  if ((do_row | q_row | k_row | v_row | o_row | dq_row | dk_row | dv_row) % 8) return (int)cudaErrorInvalidValue;
  if (((uintptr_t)dO | (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o | (uintptr_t)dq | (uintptr_t)dk |
       (uintptr_t)dv | (uintptr_t)workspace) & 15)
    return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KV_SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Q_SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(flash_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int Tpad = (Tq + 127) / 128 * 128;
  float* delta_pad = (float*)workspace;
  float* lse2_pad = delta_pad + (int64_t)H * Tpad;
  uint8_t* stat_tiles = (uint8_t*)(lse2_pad + (int64_t)H * Tpad);
  {
    const int64_t warps = (int64_t)Tpad * H;
    const int threads = 256;
    const int64_t blocks = (warps * 32 + threads - 1) / threads;
    prep_kernel<<<(unsigned)blocks, threads, 0, st>>>((const __nv_bfloat16*)dO, (const __nv_bfloat16*)o, lse, delta_pad,
                                                      lse2_pad, stat_tiles, 1.f / scale, Tq, Tpad, H, do_row, o_row);
  }
  CUtensorMap tQ, tDO, tK, tV, tDQ, tDK, tDV;
  int r;
  if ((r = make_tmap_3d_bf16(&tQ, q, HD, H, Tq, HD * 2, q_row * 2, 64, 1, BIG))) return 770000 + r;
  if ((r = make_tmap_3d_bf16(&tDO, dO, HD, H, Tq, HD * 2, do_row * 2, 64, 1, BIG))) return 770000 + r;
  if ((r = make_tmap_3d_bf16(&tK, k, HD, Hkv, Tk, HD * 2, k_row * 2, 64, 1, BIG))) return 780000 + r;
  if ((r = make_tmap_3d_bf16(&tV, v, HD, Hkv, Tk, HD * 2, v_row * 2, 64, 1, BIG))) return 780000 + r;
  if ((r = make_tmap_3d_bf16(&tDQ, dq, HD, H, Tq, HD * 2, dq_row * 2, 64, 1, BIG))) return 790000 + r;
  if ((r = make_tmap_3d_bf16(&tDK, dk, HD, Hkv, Tk, HD * 2, dk_row * 2, 64, 1, BIG))) return 790000 + r;
  if ((r = make_tmap_3d_bf16(&tDV, dv, HD, Hkv, Tk, HD * 2, dv_row * 2, 64, 1, BIG))) return 790000 + r;
  dim3 gkv((Tk + BIG - 1) / BIG, Hkv);
  if (g_bwd_variant != 1) {
    float* dq_acc = (float*)(stat_tiles + (int64_t)H * (Tpad / BLK) * STAT_BYTES);
    cudaError_t e = cudaMemsetAsync(dq_acc, 0, (size_t)H * Tpad * HD * sizeof(float), st);
    if (e != cudaSuccess) return (int)e;
    flash_bwd_fused_kernel<<<gkv, NUM_THREADS, F_SMEM_TOTAL, st>>>(tQ, tDO, tK, tV, tDK, tDV, stat_tiles, dq_acc, Tq, Tk, Tpad, H, Hkv,
                                                                   causal, scale, err, sk, sv);
    DqDests dd;
    memset(&dd, 0, sizeof(dd));
    for (int d = 0; d < n_split; ++d) dd.p[d] = (__nv_bfloat16*)dq_split[d];
    const int64_t items = (int64_t)Tq * H * (HD / 8);
    dq_convert_kernel<<<(unsigned)((items + 255) / 256), 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dq, dd, n_split > 0 ? split_rows : 0,
                                                                        dq_row, Tq, Tpad, H, scale);
    return (int)cudaGetLastError();
  }
  flash_bwd_dkdv_kernel<<<gkv, NUM_THREADS, KV_SMEM_TOTAL, st>>>(tQ, tDO, tK, tV, tDK, tDV, stat_tiles, Tq, Tk,
                                                                 Tpad, H, Hkv, causal, scale, err, g_bwd_trace, sk, sv);
  dim3 gq((Tq + BIG - 1) / BIG, H);
  flash_bwd_dq_kernel<<<gq, NUM_THREADS, Q_SMEM_TOTAL, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)dO, q_row, do_row, tK, tV, tDQ, lse2_pad, delta_pad, Tq, Tk, Tpad, H,
                                                             Hkv, causal, scale, err, sq, g_bwd_trace ? g_bwd_trace + 48 * 8 : nullptr);
  return (int)cudaGetLastError();
}
