// Attention backward for sm_100a (head_dim 128, bf16, GQA): dQ, dK, dV from (dO, Q, K, V, O, LSE).
//
// The reference gets this from flash_attn_2_cuda.bwd through autograd (reference
// decoder/odysseus.py:256-263; its ring dependency calls the same kernel per block).  Here it is three
// kernels built on tcgen05 / TMEM / TMA:
//
//   prep   : delta[h,t] = sum_d dO*O, and LSE converted to the exp2 domain, both padded to 64 rows.
//   dkdv   : one CTA per (128-row KV tile, kv head).  K and V stay in shared memory; 64-row blocks of Q
//            and dO stream through a TMA ring.  S^T = K Q^T and dP^T = V dO^T land in TMEM (double
//            buffered, kv rows on lanes), eight warps (two per lane quarter, 32 columns each) turn them into
//            P^T and dS^T (bf16, written back over
//            the same TMEM columns) and the tensor core accumulates dV += P^T dO, dK += dS^T Q in TMEM
//            (2*64 + 2*64 + 128 + 128 = 512 columns).  Query heads sharing the kv head are looped inside.
//   dq     : one CTA per (128-row query tile, head).  Q and dO stay in shared memory; 64-row blocks of K
//            and V stream.  S = Q K^T, dP = dO V^T, dS (bf16 in TMEM) and dQ += dS K.
//
// Splitting dQ from dK/dV recomputes S and dP once more but needs no atomics and is deterministic.
// Gradients are written with TMA stores through row-pitched tensor maps, so dq/dk/dv may be slices
// of one packed [T, hq + 2 hkv, 128] gradient tensor.
#include "ody_kernels.h"
#include "sm100.cuh"

namespace ody {
namespace bwd {

constexpr int HD = 128;
constexpr int BIG = 128;                         // resident tile rows
constexpr int BLK = 64;                          // streamed block rows
constexpr int BIG_BYTES = BIG * HD * 2;          // 32 KB (two halves of [128 x 128 B])
constexpr int BIG_HALF = BIG_BYTES / 2;
constexpr int BLK_BYTES = BLK * HD * 2;          // 16 KB (two halves of [64 x 128 B])
constexpr int BLK_HALF = BLK_BYTES / 2;
constexpr int STAGES = 3;
constexpr int STAT_BYTES = 2 * BLK * 4;          // lse2 + delta of one 64-row block
constexpr int NUM_THREADS = 320;             // TMA warp, MMA warp, 8 softmax warps (two per TMEM lane quarter)
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
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
// delta_pad / lse2_pad: [H, Tpad] fp32, Tpad multiple of 64; rows >= T are zero.
__global__ void prep_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                            const float* __restrict__ lse, float* __restrict__ delta_pad, float* __restrict__ lse2_pad,
                            int T, int Tpad, int H, int64_t do_row, int64_t o_row) {
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= Tpad * H) return;
  const int t = warp_global / H, h = warp_global % H;
  float s = 0.f, l2 = 0.f;
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
    l2 = lse[(int64_t)h * T + t] * LOG2E;
  }
  if (lane == 0) {
    delta_pad[(int64_t)h * Tpad + t] = s;
    lse2_pad[(int64_t)h * Tpad + t] = l2;
  }
}

// ------------------------------------------------------------------------------------------- dK / dV
struct BarsKV {
  uint64_t kv_full;
  uint64_t qd_full[STAGES], qd_empty[STAGES];
  uint64_t s_full[2], p_full[2];
  uint64_t acc_done, drain;
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int KV_SMEM_TILES = 2 * BIG_BYTES + STAGES * (2 * BLK_BYTES + STAT_BYTES);
constexpr int KV_SMEM_TOTAL = KV_SMEM_TILES + 256 + 1024;
// TMEM columns: S^T(b) at b*64, dP^T(b) at 128 + b*64 (P^T / dS^T overwrite their first 32 columns), dV 256, dK 384

// Optional redirection of an output: rows [d * rows, (d + 1) * rows) go to tensor map m[d] instead of the
// kernel's own output map (another rank's buffer: the Ulysses head->sequence exchange of the gradient).
struct SplitMaps {
  CUtensorMap m[8];
  int rows;     // 0 = unused
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ64, const __grid_constant__ CUtensorMap tmDO64,
                      const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV,
                      const float* __restrict__ lse2_pad, const float* __restrict__ delta_pad, int Tq, int Tk, int Tq_pad,
                      int H, int Hkv, int causal, float scale, int* __restrict__ err, long long* __restrict__ dbg,
                      const __grid_constant__ SplitMaps dk_split, const __grid_constant__ SplitMaps dv_split) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + BIG_BYTES;
  uint8_t* sStage = smem + 2 * BIG_BYTES;                 // per stage: Q block | dO block
  uint8_t* sStat = sStage + STAGES * 2 * BLK_BYTES;       // per stage: lse2[64] | delta[64]
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
    for (int s = 0; s < STAGES; ++s) { mbar_init(&bars->qd_full[s], 1); mbar_init(&bars->qd_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&bars->s_full[b], 1); mbar_init(&bars->p_full[b], 256); }
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

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bars->kv_full, 2 * BIG_BYTES);
      tma_load_3d(sK, &tmK, 0, kvh, kv0, &bars->kv_full);
      tma_load_3d(sK + BIG_HALF, &tmK, 64, kvh, kv0, &bars->kv_full);
      tma_load_3d(sV, &tmV, 0, kvh, kv0, &bars->kv_full);
      tma_load_3d(sV + BIG_HALF, &tmV, 64, kvh, kv0, &bars->kv_full);
      int stage = 0; uint32_t phase = 0;
      for (int it = 0; it < total; ++it) {
        const int head = kvh * G + it / per_head;
        const int qrow = (i0 + it % per_head) * BLK;
        if (!mbar_wait(&bars->qd_empty[stage], phase ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
        uint8_t* sQ = sStage + stage * 2 * BLK_BYTES;
        uint8_t* sD = sQ + BLK_BYTES;
        float* st = (float*)(sStat + stage * STAT_BYTES);
        mbar_expect_tx(&bars->qd_full[stage], 2 * BLK_BYTES + STAT_BYTES);
        tma_load_3d(sQ, &tmQ64, 0, head, qrow, &bars->qd_full[stage]);
        tma_load_3d(sQ + BLK_HALF, &tmQ64, 64, head, qrow, &bars->qd_full[stage]);
        tma_load_3d(sD, &tmDO64, 0, head, qrow, &bars->qd_full[stage]);
        tma_load_3d(sD + BLK_HALF, &tmDO64, 64, head, qrow, &bars->qd_full[stage]);
        bulk_load_1d(st, lse2_pad + (int64_t)head * Tq_pad + qrow, BLK * 4, &bars->qd_full[stage]);
        bulk_load_1d(st + BLK, delta_pad + (int64_t)head * Tq_pad + qrow, BLK * 4, &bars->qd_full[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t IDESC_S = make_idesc_bf16(BIG, BLK, 0, 0);
      constexpr uint32_t IDESC_ACC = make_idesc_bf16(BIG, HD, 0, 1);
      bool ok = mbar_wait(&bars->kv_full, 0, abort_flag, err, ODY_ERR_TIMEOUT_FULL);
      const uint64_t kdesc0 = make_smem_desc(smem_u32(sK), 16, 1024), vdesc0 = make_smem_desc(smem_u32(sV), 16, 1024);
      const uint64_t stage_k0 = make_smem_desc(smem_u32(sStage), 16, 1024);            // K-major view of a streamed block
      const uint64_t stage_mn0 = make_smem_desc(smem_u32(sStage), BLK_HALF, 1024);     // MN-major view (B of dV / dK)
      int stage = 0; uint32_t phase = 0;          // ring position of the next S/dP issue
      int stage2 = 0;                             // ring position of the next dV/dK issue
      const bool trace = dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
      auto issue_s = [&](int it) -> bool {
        if (trace && it < 48) dbg[it * 8 + 0] = clock64();                 // MMA thread starts on S/dP(it)
        if (!mbar_wait(&bars->qd_full[stage], phase, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) return false;
        if (trace && it < 48) dbg[it * 8 + 1] = clock64();                 // Q/dO block landed
        tc_fence_after();
        const int b = it & 1;
        const uint64_t q0d = desc_advance(stage_k0, stage * 2 * BLK_BYTES), d0d = desc_advance(q0d, BLK_BYTES);
        // S^T and dP^T alternate so consecutive instructions never accumulate into the same TMEM tile
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offA = (kk >> 2) * BIG_HALF + (kk & 3) * 32, offB = (kk >> 2) * BLK_HALF + (kk & 3) * 32;
          umma_ss(tmem + b * 64, desc_advance(kdesc0, offA), desc_advance(q0d, offB), IDESC_S, kk > 0 ? 1u : 0u);
          umma_ss(tmem + 128 + b * 64, desc_advance(vdesc0, offA), desc_advance(d0d, offB), IDESC_S, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->s_full[b]);
        if (trace && it < 48) dbg[it * 8 + 2] = clock64();                 // S/dP(it) issued
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
        return true;
      };
      if (ok && total > 0) ok = issue_s(0);
      for (int it = 0; it < total && ok; ++it) {
        if (it + 1 < total && !issue_s(it + 1)) { ok = false; break; }
        const int b = it & 1;
        if (!mbar_wait(&bars->p_full[b], (it >> 1) & 1, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        if (trace && it < 48) dbg[it * 8 + 3] = clock64();                 // MMA thread saw P(it)
        tc_fence_after();
        const uint64_t qmn = desc_advance(stage_mn0, stage2 * 2 * BLK_BYTES), dmn = desc_advance(qmn, BLK_BYTES);
        const uint32_t acc0 = it > 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk) {   // dV += P^T dO and dK += dS^T Q, alternating
          umma_ts(tmem + 256, tmem + b * 64 + kk * 8, desc_advance(dmn, kk * 2048), IDESC_ACC, kk > 0 ? 1u : acc0);
          umma_ts(tmem + 384, tmem + 128 + b * 64 + kk * 8, desc_advance(qmn, kk * 2048), IDESC_ACC, kk > 0 ? 1u : acc0);
        }
        umma_commit(&bars->qd_empty[stage2]);
        if (trace && it < 48) dbg[it * 8 + 4] = clock64();                 // dV/dK(it) issued
        if (++stage2 == STAGES) stage2 = 0;
      }
      if (ok) umma_commit(&bars->acc_done);
      else {
        umma_commit(&bars->drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(&bars->drain, 0) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
      }
    }
  } else {
    const int q = warp & 3;                               // TMEM lane quarter
    const int hf = (warp - 2) >> 2;                       // which 32 of the block's 64 query columns this warp handles
    const int r = q * 32 + lane;                          // kv row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const float sl2 = scale * LOG2E;
    bool ok = true;
    int stage = 0; uint32_t phase = 0;
    for (int it = 0; it < total; ++it) {
      const int b = it & 1;
      const int qrow0 = (i0 + it % per_head) * BLK + hf * 32;
      const bool strace = dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 64 && it < 48;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[b], (it >> 1) & 1, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL));
      if (strace) dbg[it * 8 + 5] = clock64();                             // softmax saw S(it)
      // s_full implies qd_full[stage] completed earlier (the MMAs consumed it); the stats are in smem
      const float* st = (const float*)(sStat + stage * STAT_BYTES) + hf * 32;
      uint32_t sv[32], dp[32];
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32(tmem + b * 64 + hf * 32 + lane_off, sv);
        tmem_ld_32x32(tmem + 128 + b * 64 + hf * 32 + lane_off, dp);
        tmem_ld_wait();
      }
      // P^T / dS^T are written over the first 32 columns of S^T / dP^T: the other warp of this lane quarter
      // must have read its inputs before either of us stores; the two also agree here on leaving the loop
      if (!named_barrier_and(4 + q, 64, ok)) { ok = false; break; }
      if (strace) dbg[it * 8 + 6] = clock64();                             // loaded + pair barrier
      const bool diag = causal && (qrow0 < kv0 + BIG);     // some (q, kv) pairs of this half block are masked
      uint32_t pp[16], ds[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float4 stl = *reinterpret_cast<const float4*>(st + (c >> 1) * 4);
        const float4 std_ = *reinterpret_cast<const float4*>(st + BLK + (c >> 1) * 4);
        const float l0 = (c & 1) ? stl.z : stl.x, l1 = (c & 1) ? stl.w : stl.y;
        const float d0 = (c & 1) ? std_.z : std_.x, d1 = (c & 1) ? std_.w : std_.y;
        float p0 = fast_exp2(__uint_as_float(sv[2 * c]) * sl2 - l0);
        float p1 = fast_exp2(__uint_as_float(sv[2 * c + 1]) * sl2 - l1);
        if (diag) {
          if (qrow0 + 2 * c < kv0 + r) p0 = 0.f;
          if (qrow0 + 2 * c + 1 < kv0 + r) p1 = 0.f;
        }
        pp[c] = pack_bf16(p0, p1);
        ds[c] = pack_bf16(p0 * (__uint_as_float(dp[2 * c]) - d0) * scale, p1 * (__uint_as_float(dp[2 * c + 1]) - d1) * scale);
      }
      tmem_st_32x16(tmem + b * 64 + hf * 16 + lane_off, pp);
      tmem_st_32x16(tmem + 128 + b * 64 + hf * 16 + lane_off, ds);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->p_full[b]);
      if (strace) dbg[it * 8 + 7] = clock64();                             // P(it) published
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
    (void)phase;
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_done, 0, abort_flag, err, ODY_ERR_TIMEOUT_MISC));
    if (ok) {
      tc_fence_after();
      // dV -> sV region, dK -> sK region (both dead now), bf16, swizzled for the TMA store; this warp converts
      // output columns [hf * 64, hf * 64 + 64), which is exactly one 64-column half of the staging tile
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        uint8_t* dst = (which == 0 ? sV : sK) + hf * BIG_HALF;
        const uint32_t col = (which == 0 ? 256 : 384) + hf * 64;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[16];
          tmem_ld_32x16(tmem + col + lane_off + c * 16, o);
          tmem_ld_wait();
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
    if (ok && warp == 2 && lane == 0 && !*abort_flag) {
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

// ------------------------------------------------------------------------------------------- dQ
struct BarsQ {
  uint64_t qd_full;
  uint64_t kv_full[STAGES], kv_empty[STAGES];
  uint64_t s_full[2], p_full[2];
  uint64_t acc_done, drain;
  uint32_t tmem_base;
  int abort_flag;
};
constexpr int Q_SMEM_TILES = 2 * BIG_BYTES + STAGES * 2 * BLK_BYTES;
constexpr int Q_SMEM_TOTAL = Q_SMEM_TILES + 256 + 1024;
// TMEM columns: S(b) at b*64 (dS overwrites its first 32 columns), dP(b) at 128 + b*64, dQ at 256

__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ CUtensorMap tmK64, const __grid_constant__ CUtensorMap tmV64,
                    const __grid_constant__ CUtensorMap tmDQ, const float* __restrict__ lse2_pad,
                    const float* __restrict__ delta_pad, int Tq, int Tk, int Tq_pad, int H, int Hkv, int causal,
                    float scale, int* __restrict__ err, const __grid_constant__ SplitMaps dq_split) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sD = smem + BIG_BYTES;
  uint8_t* sStage = smem + 2 * BIG_BYTES;                 // per stage: K block | V block
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
    mbar_init(&bars->qd_full, 1);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&bars->kv_full[s], 1); mbar_init(&bars->kv_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&bars->s_full[b], 1); mbar_init(&bars->p_full[b], 256); }
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

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bars->qd_full, 2 * BIG_BYTES);
      tma_load_3d(sQ, &tmQ, 0, head, q0, &bars->qd_full);
      tma_load_3d(sQ + BIG_HALF, &tmQ, 64, head, q0, &bars->qd_full);
      tma_load_3d(sD, &tmDO, 0, head, q0, &bars->qd_full);
      tma_load_3d(sD + BIG_HALF, &tmDO, 64, head, q0, &bars->qd_full);
      int stage = 0; uint32_t phase = 0;
      for (int it = 0; it < total; ++it) {
        if (!mbar_wait(&bars->kv_empty[stage], phase ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
        uint8_t* sK = sStage + stage * 2 * BLK_BYTES;
        uint8_t* sV = sK + BLK_BYTES;
        mbar_expect_tx(&bars->kv_full[stage], 2 * BLK_BYTES);
        tma_load_3d(sK, &tmK64, 0, kvh, it * BLK, &bars->kv_full[stage]);
        tma_load_3d(sK + BLK_HALF, &tmK64, 64, kvh, it * BLK, &bars->kv_full[stage]);
        tma_load_3d(sV, &tmV64, 0, kvh, it * BLK, &bars->kv_full[stage]);
        tma_load_3d(sV + BLK_HALF, &tmV64, 64, kvh, it * BLK, &bars->kv_full[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t IDESC_S = make_idesc_bf16(BIG, BLK, 0, 0);
      constexpr uint32_t IDESC_ACC = make_idesc_bf16(BIG, HD, 0, 1);
      bool ok = mbar_wait(&bars->qd_full, 0, abort_flag, err, ODY_ERR_TIMEOUT_FULL);
      const uint64_t qdesc0 = make_smem_desc(smem_u32(sQ), 16, 1024), ddesc0 = make_smem_desc(smem_u32(sD), 16, 1024);
      const uint64_t stage_k0 = make_smem_desc(smem_u32(sStage), 16, 1024);
      const uint64_t stage_mn0 = make_smem_desc(smem_u32(sStage), BLK_HALF, 1024);
      int stage = 0; uint32_t phase = 0;
      int stage2 = 0;
      auto issue_s = [&](int it) -> bool {
        if (!mbar_wait(&bars->kv_full[stage], phase, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const int b = it & 1;
        const uint64_t k0d = desc_advance(stage_k0, stage * 2 * BLK_BYTES), v0d = desc_advance(k0d, BLK_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offA = (kk >> 2) * BIG_HALF + (kk & 3) * 32, offB = (kk >> 2) * BLK_HALF + (kk & 3) * 32;
          umma_ss(tmem + b * 64, desc_advance(qdesc0, offA), desc_advance(k0d, offB), IDESC_S, kk > 0 ? 1u : 0u);
          umma_ss(tmem + 128 + b * 64, desc_advance(ddesc0, offA), desc_advance(v0d, offB), IDESC_S, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->s_full[b]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
        return true;
      };
      if (ok && total > 0) ok = issue_s(0);
      for (int it = 0; it < total && ok; ++it) {
        if (it + 1 < total && !issue_s(it + 1)) { ok = false; break; }
        const int b = it & 1;
        if (!mbar_wait(&bars->p_full[b], (it >> 1) & 1, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint64_t kmn = desc_advance(stage_mn0, stage2 * 2 * BLK_BYTES);
        const uint32_t acc0 = it > 0 ? 1u : 0u;
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk)   // dQ += dS K
          umma_ts(tmem + 256, tmem + b * 64 + kk * 8, desc_advance(kmn, kk * 2048), IDESC_ACC, kk > 0 ? 1u : acc0);
        umma_commit(&bars->kv_empty[stage2]);
        if (++stage2 == STAGES) stage2 = 0;
      }
      if (ok) umma_commit(&bars->acc_done);
      else {
        umma_commit(&bars->drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(&bars->drain, 0) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
      }
    }
  } else {
    const int q = warp & 3;
    const int hf = (warp - 2) >> 2;                       // which 32 of the block's 64 key columns this warp handles
    const int r = q * 32 + lane;                          // query row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const float sl2 = scale * LOG2E;
    const int64_t srow = (int64_t)head * Tq_pad + q0 + r;  // Tq_pad is a multiple of 128: every tile row has an entry
    const float my_lse2 = lse2_pad[srow];
    const float my_delta = delta_pad[srow];
    bool ok = true;
    for (int it = 0; it < total; ++it) {
      const int b = it & 1;
      const int kvb0 = it * BLK + hf * 32;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[b], (it >> 1) & 1, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL));
      uint32_t sv[32], dp[32];
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32(tmem + b * 64 + hf * 32 + lane_off, sv);
        tmem_ld_32x32(tmem + 128 + b * 64 + hf * 32 + lane_off, dp);
        tmem_ld_wait();
      }
      // dS overwrites S's first 32 columns: both warps of the quarter have loaded; they also agree on leaving
      if (!named_barrier_and(4 + q, 64, ok)) { ok = false; break; }
      const bool diag = causal && (kvb0 + 31 > q0);
      const bool tail = kvb0 + 32 > Tk;
      uint32_t ds[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        float p0 = fast_exp2(__uint_as_float(sv[2 * c]) * sl2 - my_lse2);
        float p1 = fast_exp2(__uint_as_float(sv[2 * c + 1]) * sl2 - my_lse2);
        if (diag) {
          if (kvb0 + 2 * c > q0 + r) p0 = 0.f;
          if (kvb0 + 2 * c + 1 > q0 + r) p1 = 0.f;
        }
        if (tail) {
          if (kvb0 + 2 * c >= Tk) p0 = 0.f;
          if (kvb0 + 2 * c + 1 >= Tk) p1 = 0.f;
        }
        ds[c] = pack_bf16(p0 * (__uint_as_float(dp[2 * c]) - my_delta) * scale,
                          p1 * (__uint_as_float(dp[2 * c + 1]) - my_delta) * scale);
      }
      tmem_st_32x16(tmem + b * 64 + hf * 16 + lane_off, ds);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->p_full[b]);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_done, 0, abort_flag, err, ODY_ERR_TIMEOUT_MISC));
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[16];
        tmem_ld_32x16(tmem + 256 + hf * 64 + lane_off + c * 16, o);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          uint4 v4;
          v4.x = pack_bf16(__uint_as_float(o[8 * t + 0]), __uint_as_float(o[8 * t + 1]));
          v4.y = pack_bf16(__uint_as_float(o[8 * t + 2]), __uint_as_float(o[8 * t + 3]));
          v4.z = pack_bf16(__uint_as_float(o[8 * t + 4]), __uint_as_float(o[8 * t + 5]));
          v4.w = pack_bf16(__uint_as_float(o[8 * t + 6]), __uint_as_float(o[8 * t + 7]));
          const int chunk = c * 2 + t;
          *reinterpret_cast<uint4*>(sQ + hf * BIG_HALF + r * 128 + ((chunk ^ (r & 7)) << 4)) = v4;
        }
      }
      fence_proxy_async_smem();
    }
    tc_fence_before();
    named_barrier(1, 256);
    if (ok && warp == 2 && lane == 0 && !*abort_flag) {
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
// Optional per-block timeline of CTA (0,0) of the dK/dV kernel: 48 x 8 SM-clock stamps (see the kernel).
extern "C" void ody_flash_bwd_set_trace(long long* buf) { g_bwd_trace = buf; }

extern "C" int64_t ody_flash_bwd_workspace_bytes(int Tq, int H) {
  const int64_t Tpad = ((int64_t)Tq + 127) / 128 * 128;
  return 2 * (int64_t)H * Tpad * 4;
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
    configured = true;
  }
  const int Tpad = (Tq + 127) / 128 * 128;
  float* delta_pad = (float*)workspace;
  float* lse2_pad = delta_pad + (int64_t)H * Tpad;
  {
    const int64_t warps = (int64_t)Tpad * H;
    const int threads = 256;
    const int64_t blocks = (warps * 32 + threads - 1) / threads;
    prep_kernel<<<(unsigned)blocks, threads, 0, st>>>((const __nv_bfloat16*)dO, (const __nv_bfloat16*)o, lse, delta_pad,
                                                      lse2_pad, Tq, Tpad, H, do_row, o_row);
  }
  CUtensorMap tQ, tDO, tK, tV, tQ64, tDO64, tK64, tV64, tDQ, tDK, tDV;
  int r;
  if ((r = make_tmap_3d_bf16(&tQ, q, HD, H, Tq, HD * 2, q_row * 2, 64, 1, BIG))) return 770000 + r;
  if ((r = make_tmap_3d_bf16(&tDO, dO, HD, H, Tq, HD * 2, do_row * 2, 64, 1, BIG))) return 770000 + r;
  if ((r = make_tmap_3d_bf16(&tQ64, q, HD, H, Tq, HD * 2, q_row * 2, 64, 1, BLK))) return 770000 + r;
  if ((r = make_tmap_3d_bf16(&tDO64, dO, HD, H, Tq, HD * 2, do_row * 2, 64, 1, BLK))) return 770000 + r;
  if ((r = make_tmap_3d_bf16(&tK, k, HD, Hkv, Tk, HD * 2, k_row * 2, 64, 1, BIG))) return 780000 + r;
  if ((r = make_tmap_3d_bf16(&tV, v, HD, Hkv, Tk, HD * 2, v_row * 2, 64, 1, BIG))) return 780000 + r;
  if ((r = make_tmap_3d_bf16(&tK64, k, HD, Hkv, Tk, HD * 2, k_row * 2, 64, 1, BLK))) return 780000 + r;
  if ((r = make_tmap_3d_bf16(&tV64, v, HD, Hkv, Tk, HD * 2, v_row * 2, 64, 1, BLK))) return 780000 + r;
  if ((r = make_tmap_3d_bf16(&tDQ, dq, HD, H, Tq, HD * 2, dq_row * 2, 64, 1, BIG))) return 790000 + r;
  if ((r = make_tmap_3d_bf16(&tDK, dk, HD, Hkv, Tk, HD * 2, dk_row * 2, 64, 1, BIG))) return 790000 + r;
  if ((r = make_tmap_3d_bf16(&tDV, dv, HD, Hkv, Tk, HD * 2, dv_row * 2, 64, 1, BIG))) return 790000 + r;
  dim3 gkv((Tk + BIG - 1) / BIG, Hkv);
  flash_bwd_dkdv_kernel<<<gkv, NUM_THREADS, KV_SMEM_TOTAL, st>>>(tQ64, tDO64, tK, tV, tDK, tDV, lse2_pad, delta_pad, Tq, Tk,
                                                                 Tpad, H, Hkv, causal, scale, err, g_bwd_trace, sk, sv);
  dim3 gq((Tq + BIG - 1) / BIG, H);
  flash_bwd_dq_kernel<<<gq, NUM_THREADS, Q_SMEM_TOTAL, st>>>(tQ, tDO, tK64, tV64, tDQ, lse2_pad, delta_pad, Tq, Tk, Tpad, H,
                                                             Hkv, causal, scale, err, sq);
  return (int)cudaGetLastError();
}
