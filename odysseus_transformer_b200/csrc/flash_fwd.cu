// Causal / full softmax attention forward for sm_100a (head_dim 128, bf16, GQA), with log-sum-exp.
//
// The reference reaches FlashAttention-2 (an sm80 mma.sync design) through HF's
// _flash_attention_forward (reference decoder/odysseus.py:256-263) and through its ring / Ulysses
// dependencies.  This kernel is written for the Blackwell execution model instead:
//
//   * one CTA per (128-row query tile, head); K/V blocks of 128 rows stream through a 2-stage TMA ring;
//   * S = Q K^T and O += P V are tcgen05.mma instructions issued by one thread; S (double buffered), the
//     bf16 probabilities P (double buffered, fed back as the TMEM A operand) and the fp32 O accumulator
//     live in TMEM (2*128 + 2*64 + 128 = 512 columns);
//   * eight softmax warps, two threads per query row (64 of the 128 key columns each, so every scheduler
//     has two warps to interleave), read S straight from TMEM, exchange their partial row maxima through
//     shared memory, work in the exp2 domain and rescale O lazily: the running maximum used for
//     exponentiation only moves when it would grow by more than 2^8, so the O read-modify-write is rare;
//   * S = Q K^T and O += P V are issued by two different warps: a single thread sustains only about one
//     tcgen05.mma per ~85 cycles, and with 64-cycle instructions one issuer would leave the tensor core
//     idle a third of the time.  Q K^T of block j+2 goes out as soon as the softmax warps have loaded
//     S of block j into registers.
//
// q [Tq, H, 128], k/v [Tk, Hkv, 128] with arbitrary row pitch; out [Tq, H, 128] bf16; lse [H, Tq] fp32
// (natural log).  causal requires Tq == Tk (row i sees keys 0..i).
#include "ody_kernels.h"
#include "sm100.cuh"
#include "peer_comm.cuh"

// Of every ODY_FWD_POLY_DEN column pairs, the first ODY_FWD_POLY_NUM take their exponentials on the FMA pipe
// (exp2_poly2) instead of the special-function unit.  Measured on B200: any mix is a few percent slower than
// all-MUFU - the softmax warps are bound by the latency of their dependent chains, not by either pipe - so it is off.
#ifndef ODY_FWD_POLY_NUM
#define ODY_FWD_POLY_NUM 0
#define ODY_FWD_POLY_DEN 2
#endif

namespace ody {
namespace fwd {

constexpr int BM = 128, BN = 128, HD = 128;
constexpr int TILE_BYTES = 128 * HD * 2;     // 32 KB: two 64-column halves of [128 rows x 128 B]
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int KV_STAGES = 2;
constexpr int SMEM_TILES = TILE_BYTES * (1 + 2 * KV_STAGES);
constexpr int SMEM_TOTAL = SMEM_TILES + 2560 + 1024;
// Warp roles, grouped by warpgroup so that the PUSH variant can move registers between them:
//   0 TMA producer, 1 Q K^T issuer, 2 P V issuer, 3 idle | 4..11 softmax (two per TMEM lane quarter) | 12..15 comm (PUSH only)
constexpr int NUM_THREADS = 384;
constexpr int NUM_THREADS_PUSH = NUM_THREADS + gc::COMM_THREADS;
// Register split of the PUSH variant by setmaxnreg: 512 threads are launched with 128 registers each; the split
// must fit inside that allocation or the increase never returns.
constexpr int REGS_ISSUE = 56, REGS_MATH = 176, REGS_COMM = 104;
static_assert(128 * REGS_ISSUE + 256 * REGS_MATH + 128 * REGS_COMM <= NUM_THREADS_PUSH * 128, "setmaxnreg split exceeds the CTA's registers");
constexpr uint32_t COL_S = 0, COL_O = 256, COL_P = 384;

// Optional second destination of the output: rows [d * rows, (d + 1) * rows) also go to tensor map m[d]
// (another rank's buffer: the Ulysses head->sequence exchange happens in this epilogue).
struct SplitMaps {
  CUtensorMap m[8];
  int rows;     // 0 = unused
};

struct Bars {
  uint64_t q_full;
  uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
  uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
  uint64_t s_full[2], s_free[2], p_full[2], pv_done[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
  float pmax[2][2][128];      // [parity][column half][row]: partial row maxima (and, at the end, row sums)
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

// PUSH: four extra comm warps in CTAs 0..push_ctas-1 store this rank's K/V shard into the gathered
// buffers of the ring peers named by `pp` while the attention tiles run (ring attention: the kernel of
// ring step s delivers the shard that the peer s+1 places downstream needs for its step s+1).
template <bool PUSH>
__global__ void __launch_bounds__(PUSH ? NUM_THREADS_PUSH : NUM_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                 float* __restrict__ lse, int Tq, int Tk, int H, int Hkv, int causal, float scale,
                 int* __restrict__ err, long long* __restrict__ dbg, const __grid_constant__ gc::GatherParams pp,
                 int push_ctas, const __grid_constant__ SplitMaps osplit) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE_BYTES;
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;
  Bars* bars = (Bars*)(smem + SMEM_TILES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_q_tiles = (Tq + BM - 1) / BM;
  const int qt = causal ? (num_q_tiles - 1 - (int)blockIdx.x) : (int)blockIdx.x;   // heavy tiles first
  const int head = blockIdx.y;
  const int kv_head = head / (H / Hkv);
  const int q0 = qt * BM;
  const int nblk = causal ? (qt + 1) : (Tk + BN - 1) / BN;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->s_full[b], 1);
      mbar_init(&bars->s_free[b], 256);
      mbar_init(&bars->p_full[b], 256);
      mbar_init(&bars->pv_done[b], 1);
    }
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmO);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  // PUSH: 512 threads start with 128 registers each; the softmax warpgroups need more, everyone else far less
  if (warp >= 12) {
    // ------------------------------------------------------------------ comm warps (PUSH only)
    if constexpr (PUSH) {
      reg_dec<REGS_COMM>();
      const int cta = blockIdx.y * gridDim.x + blockIdx.x;
      if (cta < push_ctas) gc::comm_warps_main(pp, cta, push_ctas, 12 * 32, abort_flag, err);
    }
  } else if (warp < 4) {
   if constexpr (PUSH) reg_dec<REGS_ISSUE>();
   if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, TILE_BYTES);
      tma_load_3d(sQ, &tmQ, 0, head, q0, &bars->q_full);
      tma_load_3d(sQ + HALF_BYTES, &tmQ, 64, head, q0, &bars->q_full);
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bars->k_empty[s], ph ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&bars->k_full[s], TILE_BYTES);
        tma_load_3d(sK + s * TILE_BYTES, &tmK, 0, kv_head, j * BN, &bars->k_full[s]);
        tma_load_3d(sK + s * TILE_BYTES + HALF_BYTES, &tmK, 64, kv_head, j * BN, &bars->k_full[s]);
        if (!mbar_wait(&bars->v_empty[s], ph ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&bars->v_full[s], TILE_BYTES);
        tma_load_3d(sV + s * TILE_BYTES, &tmV, 0, kv_head, j * BN, &bars->v_full[s]);
        tma_load_3d(sV + s * TILE_BYTES + HALF_BYTES, &tmV, 64, kv_head, j * BN, &bars->v_full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ Q K^T issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = make_idesc_bf16(BM, BN, 0, 0);
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag, err, ODY_ERR_TIMEOUT_FULL);
      const uint64_t qdesc0 = make_smem_desc(smem_u32(sQ), 16, 1024);
      const uint64_t kdesc0 = make_smem_desc(smem_u32(sK), 16, 1024);
      for (int j = 0; j < nblk && ok; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const bool tr = dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && j < 48;
        if (tr) dbg[j * 8 + 0] = clock64();
        if (!mbar_wait(&bars->k_full[b], ph, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) { ok = false; break; }
        // S buffer b was last read by the softmax of block j-2
        if (j >= 2 && !mbar_wait(&bars->s_free[b], ph ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        if (tr) dbg[j * 8 + 1] = clock64();
        tc_fence_after();
        const uint64_t k0 = desc_advance(kdesc0, b * TILE_BYTES);
        umma_ss(tmem + COL_S + b * BN, qdesc0, k0, IDESC_QK, 0u);
#pragma unroll
        for (int kk = 1; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
          umma_ss(tmem + COL_S + b * BN, desc_advance(qdesc0, off), desc_advance(k0, off), IDESC_QK, 1u);
        }
        umma_commit(&bars->k_empty[b]);
        umma_commit(&bars->s_full[b]);
        if (tr) dbg[j * 8 + 2] = clock64();
      }
      if (!ok) {
        umma_commit(&bars->drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(&bars->drain, 0) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ P V issuer
    if (lane == 0) {
      constexpr uint32_t IDESC_PV = make_idesc_bf16(BM, HD, 0, 1);
      const uint64_t vdesc0 = make_smem_desc(smem_u32(sV), HALF_BYTES, 1024);
      for (int j = 0; j < nblk; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bars->p_full[b], ph, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL)) break;
        if (!mbar_wait(&bars->v_full[b], ph, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) break;
        const bool tr = dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && j < 48;
        if (tr) dbg[j * 8 + 3] = clock64();
        tc_fence_after();
        const uint64_t v0 = desc_advance(vdesc0, b * TILE_BYTES);
        const uint32_t pa = tmem + COL_P + b * 64;
        umma_ts(tmem + COL_O, pa, v0, IDESC_PV, j > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 1; kk < BN / 16; ++kk) umma_ts(tmem + COL_O, pa + kk * 8, desc_advance(v0, kk * 2048), IDESC_PV, 1u);
        umma_commit(&bars->v_empty[b]);
        umma_commit(&bars->pv_done[b]);
        if (tr) dbg[j * 8 + 4] = clock64();
      }
    }
   }   // warp 3 idles: it only keeps the warpgroups aligned
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (warps 4..11)
    if constexpr (PUSH) reg_inc<REGS_MATH>();
    const int q = warp & 3;                            // TMEM lane quarter
    const int hf = (warp - 4) >> 2;                    // key columns [hf * 64, hf * 64 + 64) of every block
    const int r = q * 32 + lane;                       // row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const float sl2 = scale * 1.4426950408889634f;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    // `ok` is kept warp-uniform; the two warps of a lane quarter agree on it at their exchange barrier, so
    // they always leave the loop in the same iteration
    for (int j = 0; j < nblk; ++j) {
      const int b = j & 1;
      const bool str_ = dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 128 && j < 48;
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[b], (j >> 1) & 1, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL));
      if (str_) dbg[j * 8 + 5] = clock64();
      uint32_t sv[64];
      float mx = -INFINITY;
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32(tmem + COL_S + b * BN + hf * 64 + lane_off, sv);
        tmem_ld_32x32(tmem + COL_S + b * BN + hf * 64 + 32 + lane_off, sv + 32);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&bars->s_free[b]);                 // S(j) is in registers: Q K^T of block j+2 may overwrite it
        const int kv0 = j * BN + hf * 64;
        if (causal && j == qt) {
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (hf * 64 + c > r) sv[c] = 0xff800000u;   // -inf
        }
        if (kv0 + 64 > Tk) {
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (kv0 + c >= Tk) sv[c] = 0xff800000u;
        }
        // partial row maximum over our 64 columns, four independent chains
        float m0 = __uint_as_float(sv[0]), m1 = __uint_as_float(sv[1]), m2 = __uint_as_float(sv[2]), m3 = __uint_as_float(sv[3]);
#pragma unroll
        for (int c = 4; c < 64; c += 4) {
          m0 = fmaxf(m0, __uint_as_float(sv[c]));
          m1 = fmaxf(m1, __uint_as_float(sv[c + 1]));
          m2 = fmaxf(m2, __uint_as_float(sv[c + 2]));
          m3 = fmaxf(m3, __uint_as_float(sv[c + 3]));
        }
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        // the two threads of a row swap partial maxima (double-buffered on the block parity)
        bars->pmax[b][hf][r] = mx;
      }
      if (!named_barrier_and(4 + q, 64, ok)) { ok = false; break; }
      if (str_) dbg[j * 8 + 6] = clock64();
      mx = fmaxf(mx, bars->pmax[b][hf ^ 1][r]);
      const float m_new = fmaxf(m_used, mx * sl2);
      const bool need = (m_new - m_used) > 8.f;      // true on the first block (m_used = -inf)
      if (j == 0) {
        m_used = m_new;
      } else if (__any_sync(0xffffffffu, need)) {
        // the running maximum moved by more than 2^8 for some row of this warp: rescale O (our 64 columns) and l
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, err, ODY_ERR_TIMEOUT_MISC));
        if (ok) {
          tc_fence_after();
          const float alpha = need ? fast_exp2(m_used - m_new) : 1.f;
          if (need) m_used = m_new;
          l *= alpha;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[16];
            tmem_ld_32x16(tmem + COL_O + hf * 64 + lane_off + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < 16; ++t) o[t] = __float_as_uint(__uint_as_float(o[t]) * alpha);
            tmem_st_32x16(tmem + COL_O + hf * 64 + lane_off + c * 16, o);
          }
          tmem_st_wait();
        }
      }
      // packed pairs: x = s * scale * log2(e) - m for two columns per instruction, two running partial sums
      const uint64_t sl2_2 = pk2(sl2, sl2), nm_2 = pk2(-m_used, -m_used);
      uint64_t rs2 = pk2(0.f, 0.f);
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float p0, p1;
        const uint64_t x2 = fma2(pk2u(sv[2 * c], sv[2 * c + 1]), sl2_2, nm_2);
        if ((c % ODY_FWD_POLY_DEN) < ODY_FWD_POLY_NUM) {
          exp2_poly2(x2, p0, p1);
        } else {
          upk2(x2, p0, p1);
          p0 = exp2_mufu(p0);
          p1 = exp2_mufu(p1);
        }
        rs2 = add2(rs2, pk2(p0, p1));
        pk[c] = pack_bf16(p0, p1);
      }
      {
        float r0, r1;
        upk2(rs2, r0, r1);
        l += r0 + r1;
      }
      if (ok && j >= 2)   // P buffer b was last read by P V of block j-2
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->pv_done[b], ((j - 2) >> 1) & 1, abort_flag, err, ODY_ERR_TIMEOUT_MISC));
      if (ok) {
        tmem_st_32x16(tmem + COL_P + b * 64 + hf * 32 + lane_off, pk);
        tmem_st_32x16(tmem + COL_P + b * 64 + hf * 32 + 16 + lane_off, pk + 16);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&bars->p_full[b]);
        if (str_) dbg[j * 8 + 7] = clock64();
      }
    }
    // epilogue: O / l -> bf16 -> swizzled smem (the Q tile is dead by now) -> TMA store; lse
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->pv_done[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, abort_flag, err, ODY_ERR_TIMEOUT_MISC));
    // the row sum is split over the two threads of a row
    bars->pmax[0][hf][r] = l;
    named_barrier(4 + q, 64);
    l += bars->pmax[0][hf ^ 1][r];
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l;
#pragma unroll
      for (int c = 0; c < 4; ++c) {                   // our 64 output columns = staging half `hf`
        uint32_t o[16];
        tmem_ld_32x16(tmem + COL_O + hf * 64 + lane_off + c * 16, o);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          uint4 v4;
          v4.x = pack_bf16(__uint_as_float(o[8 * t + 0]) * inv_l, __uint_as_float(o[8 * t + 1]) * inv_l);
          v4.y = pack_bf16(__uint_as_float(o[8 * t + 2]) * inv_l, __uint_as_float(o[8 * t + 3]) * inv_l);
          v4.z = pack_bf16(__uint_as_float(o[8 * t + 4]) * inv_l, __uint_as_float(o[8 * t + 5]) * inv_l);
          v4.w = pack_bf16(__uint_as_float(o[8 * t + 6]) * inv_l, __uint_as_float(o[8 * t + 7]) * inv_l);
          const int chunk = c * 2 + t;                // 16-byte chunk inside the 128-byte row of this half
          *reinterpret_cast<uint4*>(sQ + hf * HALF_BYTES + r * 128 + ((chunk ^ (r & 7)) << 4)) = v4;
        }
      }
      if (hf == 0 && q0 + r < Tq) lse[(int64_t)head * Tq + q0 + r] = (m_used + log2f(l)) * 0.6931471805599453f;
      fence_proxy_async_smem();
    }
    tc_fence_before();
    named_barrier(1, 256);
    if (ok && warp == 4 && lane == 0 && !*abort_flag) {
      tma_store_3d(&tmO, sQ, 0, head, q0);
      tma_store_3d(&tmO, sQ + HALF_BYTES, 64, head, q0);
      if (osplit.rows > 0) {
        const int d = q0 / osplit.rows;
        tma_store_3d(&osplit.m[d], sQ, 0, head, q0 - d * osplit.rows);
        tma_store_3d(&osplit.m[d], sQ + HALF_BYTES, 64, head, q0 - d * osplit.rows);
      }
      tma_store_commit();
      tma_store_wait<0>();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace fwd
}  // namespace ody

static long long* g_fwd_trace = nullptr;
// Optional per-block timeline (48 x 8 SM-clock stamps) of the CTA with blockIdx (0, 0).
extern "C" void ody_flash_fwd_set_trace(long long* buf) { g_fwd_trace = buf; }

// q/k/v/o: bf16, head_dim 128, element strides: *_row (token pitch), heads packed (pitch 128).
extern "C" int ody_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int Tq, int Tk, int H,
                             int Hkv, int64_t q_row, int64_t k_row, int64_t v_row, int64_t o_row, int causal,
                             float scale, int* err, cudaStream_t st) {
  return ody_flash_fwd_ex(q, k, v, o, lse, Tq, Tk, H, Hkv, q_row, k_row, v_row, o_row, causal, scale, nullptr, nullptr, 0, 0, 0,
                          err, st);
}

extern "C" int ody_flash_set_push_order(int unit_major) {
  return (int)cudaMemcpyToSymbol(ody::gc::g_push_unit_major, &unit_major, sizeof(unit_major));
}

extern "C" int ody_flash_set_peer_wait_limit(long long cycles) {
  if (cycles <= 0) return (int)cudaErrorInvalidValue;
  return (int)cudaMemcpyToSymbol(ody::gc::g_peer_spin_limit, &cycles, sizeof(cycles));
}

// Same kernel; when `push` is given, CTAs 0..push->n_cta-1 also deliver push->shard to the destinations it names.
extern "C" int ody_flash_fwd_push(const void* q, const void* k, const void* v, void* o, float* lse, int Tq, int Tk, int H,
                                  int Hkv, int64_t q_row, int64_t k_row, int64_t v_row, int64_t o_row, int causal,
                                  float scale, const OdyGatherDesc* push, int* err, cudaStream_t st) {
  return ody_flash_fwd_ex(q, k, v, o, lse, Tq, Tk, H, Hkv, q_row, k_row, v_row, o_row, causal, scale, push, nullptr, 0, 0, 0, err, st);
}

// Full form: optional push (ring) and optional split of the output rows over n_split extra destinations
// o_split[d] ([split_rows, H, 128], row pitch split_row elements; may be peer memory), split_rows % 128 == 0.
extern "C" int ody_flash_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse, int Tq, int Tk, int H,
                                int Hkv, int64_t q_row, int64_t k_row, int64_t v_row, int64_t o_row, int causal, float scale,
                                const OdyGatherDesc* push, void* const* o_split, int n_split, int split_rows,
                                int64_t split_row, int* err, cudaStream_t st) {
  using namespace ody;
  using namespace ody::fwd;
  if (Tq <= 0 || Tk <= 0 || H <= 0 || Hkv <= 0 || H % Hkv) return (int)cudaErrorInvalidValue;
  if (causal && Tq != Tk) return (int)cudaErrorInvalidValue;
  if ((q_row % 8) || (k_row % 8) || (v_row % 8) || (o_row % 8)) return (int)cudaErrorInvalidValue;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15) return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap tQ, tK, tV, tO;
  int r;
  if ((r = make_tmap_3d_bf16(&tQ, q, HD, H, Tq, HD * 2, q_row * 2, 64, 1, BM))) return 730000 + r;
  if ((r = make_tmap_3d_bf16(&tK, k, HD, Hkv, Tk, HD * 2, k_row * 2, 64, 1, BN))) return 740000 + r;
  if ((r = make_tmap_3d_bf16(&tV, v, HD, Hkv, Tk, HD * 2, v_row * 2, 64, 1, BN))) return 750000 + r;
  if ((r = make_tmap_3d_bf16(&tO, o, HD, H, Tq, HD * 2, o_row * 2, 64, 1, BM))) return 760000 + r;
  SplitMaps sm;
  memset(&sm, 0, sizeof(sm));
  if (n_split > 0) {
    if (n_split > 8 || split_rows <= 0 || (split_rows % BM) || (int64_t)split_rows * n_split < Tq || (split_row % 8)) return (int)cudaErrorInvalidValue;
    for (int d = 0; d < n_split; ++d) {
      if ((uintptr_t)o_split[d] & 15) return (int)cudaErrorInvalidValue;
      if ((r = make_tmap_3d_bf16(&sm.m[d], o_split[d], HD, H, split_rows, HD * 2, split_row * 2, 64, 1, BM))) return 770000 + r;
    }
    sm.rows = split_rows;
  }
  dim3 grid((Tq + BM - 1) / BM, H);
  if (push != nullptr) {
    gc::GatherParams pp;
    memset(&pp, 0, sizeof(pp));
    if ((r = gc::fill_gather(pp, push))) return r;
    const int ctas = (int)(grid.x * grid.y);
    if (push->n_cta <= 0 || push->n_cta > ctas) return (int)cudaErrorInvalidValue;
    flash_fwd_kernel<true><<<grid, NUM_THREADS_PUSH, SMEM_TOTAL, st>>>(tQ, tK, tV, tO, lse, Tq, Tk, H, Hkv, causal, scale, err,
                                                                       g_fwd_trace, pp, push->n_cta, sm);
  } else {
    gc::GatherParams pp;
    memset(&pp, 0, sizeof(pp));
    flash_fwd_kernel<false><<<grid, NUM_THREADS, SMEM_TOTAL, st>>>(tQ, tK, tV, tO, lse, Tq, Tk, H, Hkv, causal, scale, err,
                                                                    g_fwd_trace, pp, 0, sm);
  }
  return (int)cudaGetLastError();
}
