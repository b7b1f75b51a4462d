// Causal / full softmax attention forward for sm_100a (head_dim 128, bf16, GQA), with log-sum-exp.
//
// The reference reaches FlashAttention-2 (an sm80 mma.sync design) through HF's
// _flash_attention_forward (reference decoder/odysseus.py:256-263) and through its ring / Ulysses
// dependencies.  This kernel is written for the Blackwell execution model instead:
//
//   * one CTA per (256 query rows, head): TWO 128-row query tiles A and B that take turns on the tensor
//     core.  While the softmax warpgroup of one tile turns its scores into probabilities, the tensor core
//     runs P V and the next Q K^T of the other tile, so neither the tensor pipe nor the exponential unit
//     waits for the other (with a single tile per CTA they alternate and each idles half the time);
//   * K/V blocks of 128 rows stream through two-stage TMA rings and are used by both tiles;
//   * every MMA is a tcgen05.mma issued by ONE thread in program order: S_t = Q_t K^T (operands in shared
//     memory) and O_t += P_t V (P_t read from TMEM).  TMEM holds S_A, S_B, O_A, O_B (4 x 128 fp32 columns);
//     the bf16 probabilities P_t are written over the first 64 columns of S_t once its thread has S_t in
//     registers - the in-order tensor pipe runs Q K^T of the next block only after P V has read them (announcing
//     P in 32-key pieces so that P V could start early measured slower: four store waits instead of one);
//   * two softmax warpgroups, one thread per query row: 128 scores straight from TMEM, no exchange between
//     threads, exp2 domain, lazy rescaling of O (the running maximum used for exponentiation only moves when
//     it would grow by more than 2^8, so the O read-modify-write is rare) - and because that maximum is known
//     before the block arrives, the exponentials start at once and the block's own maximum is found on the side.  A tcgen05.commit after Q K^T of
//     block j also covers P V of block j-1, so a thread that sees S(j) may touch O without another barrier.
//
// q [Tq, H, 128], k/v [Tk, Hkv, 128] with arbitrary row pitch; out [Tq, H, 128] bf16; lse [H, Tq] fp32
// (natural log).  causal requires Tq == Tk (row i sees keys 0..i).
#include "ody_kernels.h"
#include "sm100.cuh"
#include "peer_comm.cuh"

// KS32: Q and K sit in shared memory as eight [128 rows x 32 B] slices (32-byte swizzle) instead of two
// [128 rows x 128 B] halves (128-byte swizzle), so that each Q K^T instruction reads two contiguous 4 KB blocks.
// (Moving part of the exponentials from the special-function unit to an FMA-pipe polynomial, or announcing P in four
// pieces so that P V starts early, both measured slower than this form.)

// Development aid, compiled only with -DODY_ATTN_TRACE: SM-clock stamps of one CTA's first blocks, written to a buffer
// given with ody_flash_fwd_set_trace ([64 blocks][16] int64: 0-4 softmax of tile A, 5-9 softmax of tile B, 10-13 MMA thread).
#ifdef ODY_ATTN_TRACE
__device__ long long* g_fwd_trace_buf = nullptr;
#define ODY_FWD_STAMP(cond, j, slot) do { if ((cond) && (j) < 64 && g_fwd_trace_buf) g_fwd_trace_buf[(j) * 16 + (slot)] = clock64(); } while (0)
#else
#define ODY_FWD_STAMP(cond, j, slot) do { } while (0)
#endif

namespace ody {
namespace fwd {

constexpr int BM = 128, BN = 128, HD = 128;
constexpr int CTA_ROWS = 2 * BM;             // two query tiles per CTA
constexpr int TILE_BYTES = 128 * HD * 2;     // 32 KB: two 64-column halves of [128 rows x 128 B]
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr int KV_STAGES = 2;
constexpr int SMEM_TILES = TILE_BYTES * (2 + 2 * KV_STAGES);
constexpr int SMEM_TOTAL = SMEM_TILES + 512 + 1024;
// Warp roles by warpgroup: 0 TMA producer, 1 MMA issuer, 2-3 idle | 4..7 softmax of tile A | 8..11 softmax of
// tile B | 12..15 comm (PUSH only).  Registers move between the warpgroups with setmaxnreg; the split must fit
// inside what the CTA was launched with or the increase never returns.
constexpr int NUM_THREADS = 384;
constexpr int NUM_THREADS_PUSH = NUM_THREADS + gc::COMM_THREADS;
constexpr int REGS_ISSUE = 56, REGS_MATH = 216;                            // 384 threads launched with 168 registers each
constexpr int REGS_ISSUE_PUSH = 48, REGS_MATH_PUSH = 184, REGS_COMM = 88;  // 512 threads launched with 128 each
static_assert(128 * REGS_ISSUE + 256 * REGS_MATH <= NUM_THREADS * 168, "setmaxnreg split exceeds the CTA's registers");
static_assert(128 * REGS_ISSUE_PUSH + 256 * REGS_MATH_PUSH + 128 * REGS_COMM <= NUM_THREADS_PUSH * 128, "setmaxnreg split exceeds the CTA's registers (push)");
constexpr uint32_t COL_S = 0, COL_O = 256;   // S_t at COL_S + t * 128 (P_t over its first 64 columns), O_t at COL_O + t * 128

// Optional second destination of the output: rows [d * rows, (d + 1) * rows) also go to tensor map m[d]
// (another rank's buffer: the Ulysses head->sequence exchange happens in this epilogue).
struct SplitMaps {
  CUtensorMap m[8];
  int rows;     // 0 = unused
};

struct Bars {
  uint64_t q_full[2];
  uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
  uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
  uint64_t s_full[2], p_full[2], o_done[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

// PUSH: four extra comm warps in CTAs 0..push_ctas-1 store this rank's K/V shard into the gathered
// buffers of the ring peers named by `pp` while the attention tiles run (ring attention: the kernel of
// ring step s delivers the shard that the peer s+1 places downstream needs for its step s+1).
template <bool PUSH, bool KS32>
__global__ void __launch_bounds__(PUSH ? NUM_THREADS_PUSH : NUM_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                 float* __restrict__ lse, int Tq, int Tk, int H, int Hkv, int causal, float scale,
                 int* __restrict__ err, const __grid_constant__ gc::GatherParams pp,
                 int push_ctas, const __grid_constant__ SplitMaps osplit) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                               // tile t at sQ + t * TILE_BYTES (reused as output staging)
  uint8_t* sK = smem + 2 * TILE_BYTES;
  uint8_t* sV = sK + KV_STAGES * TILE_BYTES;
  Bars* bars = (Bars*)(smem + SMEM_TILES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_pairs = (Tq + CTA_ROWS - 1) / CTA_ROWS;
  const int pair = causal ? (num_pairs - 1 - (int)blockIdx.x) : (int)blockIdx.x;    // heavy tiles first
  const int head = blockIdx.y;
  const int kv_head = head / (H / Hkv);
  const int q0 = pair * CTA_ROWS;
  const bool has_b = q0 + BM < Tq;
  const int kv_blocks = (Tk + BN - 1) / BN;
  // blocks each tile attends to: causal tile A ends on its diagonal block q0 / 128, tile B one block later
  const int nA = causal ? (q0 / BN + 1) : kv_blocks;
  const int nB = has_b ? (causal ? nA + 1 : kv_blocks) : 0;
  const int nblk = nA > nB ? nA : nB;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full[0], 1);
    mbar_init(&bars->q_full[1], 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&bars->s_full[t], 1);
      mbar_init(&bars->p_full[t], 128);
      mbar_init(&bars->o_done[t], 1);
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

  if (warp >= 12) {
    // ------------------------------------------------------------------ comm warps (PUSH only)
    if constexpr (PUSH) {
      reg_dec<REGS_COMM>();
      const int cta = blockIdx.y * gridDim.x + blockIdx.x;
      if (cta < push_ctas) gc::comm_warps_main(pp, cta, push_ctas, 12 * 32, abort_flag, err);
    }
  } else if (warp < 4) {
    reg_dec<PUSH ? REGS_ISSUE_PUSH : REGS_ISSUE>();
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        // a [128 x 128] K-major tile: two 64-column halves, or eight 16-column slices with KS32
        auto load_kmajor = [&](uint8_t* dst, const CUtensorMap* tm, int h, int row, uint64_t* bar) {
          mbar_expect_tx(bar, TILE_BYTES);
          if constexpr (KS32) {
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) tma_load_3d(dst + kk * 4096, tm, kk * 16, h, row, bar);
          } else {
            tma_load_3d(dst, tm, 0, h, row, bar);
            tma_load_3d(dst + HALF_BYTES, tm, 64, h, row, bar);
          }
        };
        load_kmajor(sQ, &tmQ, head, q0, &bars->q_full[0]);
        if (has_b) load_kmajor(sQ + TILE_BYTES, &tmQ, head, q0 + BM, &bars->q_full[1]);
        int issued_k = 0, issued_v = 0;
        for (int j = 0; j < nblk; ++j) {
          const int s = j & 1;
          const uint32_t ph = (j >> 1) & 1;
          if (!mbar_wait(&bars->k_empty[s], ph ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
          load_kmajor(sK + s * TILE_BYTES, &tmK, kv_head, j * BN, &bars->k_full[s]);
          ++issued_k;
          if (!mbar_wait(&bars->v_empty[s], ph ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) break;
          mbar_expect_tx(&bars->v_full[s], TILE_BYTES);
          tma_load_3d(sV + s * TILE_BYTES, &tmV, 0, kv_head, j * BN, &bars->v_full[s]);
          tma_load_3d(sV + s * TILE_BYTES + HALF_BYTES, &tmV, 64, kv_head, j * BN, &bars->v_full[s]);
          ++issued_v;
        }
        if (*abort_flag) {
          // somebody gave up: nobody may be consuming any more, so let the copies still in flight land before the
          // CTA's shared memory goes away (bounded)
          const long long t0 = clock64();
          for (int b = 0; b < 2; ++b) {
            const int jk = issued_k - 1 - b, jv = issued_v - 1 - b;
            while (jk >= 0 && !mbar_try_wait(&bars->k_full[jk & 1], (jk >> 1) & 1) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
            while (jv >= 0 && !mbar_try_wait(&bars->v_full[jv & 1], (jv >> 1) & 1) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
          }
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      // One issuing warp for both tiles.  Every lane runs the control flow and one elected lane issues the tcgen05
      // instructions: with warp-uniform control flow the compiler keeps descriptors and loop state in uniform registers and
      // an MMA costs a few instructions, where the same loop under `if (lane == 0)` is divergent code with many more
      // instructions per MMA.  That matters because the pipe takes a 128 x 128 x 16 instruction every 64 cycles and the
      // issuing warp shares its scheduler with softmax warps that rarely stall: measured with a probe
      // (benchmarks/mma_issue_rate.cu), the single-lane form gets an instruction out every 99 cycles next to dense
      // arithmetic warps, the elected-lane form every 64.  In this kernel the change is 1007 -> 1085 and 1161 -> 1250
      // TFLOP/s.  Measured before it and not kept: one issuing warp per tile (the tiles fall into step: both compute
      // exponentials, then both wait for the pipe; 758 TFLOP/s), a tile's chain issued from its own softmax warp with a
      // token that makes the tiles take turns (893), and pauses in the softmax warps that hand the scheduler to the
      // issuing warp (915).  The single issuer also keeps the tiles out of step, which is what lets one tile's MMAs run
      // under the other tile's exponentials.
      {
        const bool leader = elect_one();
        constexpr uint32_t IDESC_QK = make_idesc_bf16(BM, BN, 0, 0);
        constexpr uint32_t IDESC_PV = make_idesc_bf16(BM, HD, 0, 1);
        uint64_t qdesc0 = KS32 ? make_smem_desc_sw32(smem_u32(sQ)) : make_smem_desc(smem_u32(sQ), 16, 1024);
        uint64_t kdesc0 = KS32 ? make_smem_desc_sw32(smem_u32(sK)) : make_smem_desc(smem_u32(sK), 16, 1024);
        uint64_t vdesc0 = make_smem_desc(smem_u32(sV), HALF_BYTES, 1024);
        bool ok = true;
        // S_t = Q_t K(j)^T
        auto issue_qk = [&](int t, int j) {
          const uint64_t q = desc_advance(qdesc0, t * TILE_BYTES);
          const uint64_t k = desc_advance(kdesc0, (j & 1) * TILE_BYTES);
          const uint32_t d = tmem + COL_S + t * BN;
          if (leader) umma_ss(d, q, k, IDESC_QK, 0u);
#pragma unroll
          for (int kk = 1; kk < HD / 16; ++kk) {
            const uint32_t off = KS32 ? kk * 4096 : (kk >> 2) * HALF_BYTES + (kk & 3) * 32;
            if (leader) umma_ss(d, desc_advance(q, off), desc_advance(k, off), IDESC_QK, 1u);
          }
          if (leader) umma_commit(&bars->s_full[t]);
        };
        // O_t (+)= P_t V(j)
        auto issue_pv = [&](int t, int j) {
          const uint64_t v = desc_advance(vdesc0, (j & 1) * TILE_BYTES);
          const uint32_t pa = tmem + COL_S + t * BN;
          const uint32_t d = tmem + COL_O + t * HD;
          if (leader) umma_ts(d, pa, v, IDESC_PV, j > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < BN / 16; ++kk) if (leader) umma_ts(d, pa + kk * 8, desc_advance(v, kk * 2048), IDESC_PV, 1u);
        };
        ok = mbar_wait(&bars->q_full[0], 0, abort_flag, err, ODY_ERR_TIMEOUT_FULL) &&
             mbar_wait(&bars->k_full[0], 0, abort_flag, err, ODY_ERR_TIMEOUT_FULL);
        if (ok) {
          tc_fence_after();
          issue_qk(0, 0);
          if (nB > 0) {
            ok = mbar_wait(&bars->q_full[1], 0, abort_flag, err, ODY_ERR_TIMEOUT_FULL);
            if (ok) issue_qk(1, 0);
          }
          if (leader) umma_commit(&bars->k_empty[0]);
        }
        for (int j = 0; j < nblk && ok; ++j) {
          // keep the descriptor bases opaque: the compiler would otherwise hold every base + slice offset of the loop
          // in registers this thread does not have, instead of one add per MMA
          asm volatile("" : "+l"(qdesc0), "+l"(kdesc0), "+l"(vdesc0));
          const int s = j & 1, s1 = (j + 1) & 1;
          const uint32_t ph = (j >> 1) & 1, ph1 = ((j + 1) >> 1) & 1;
          bool have_v = false, have_k1 = false;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const int nt = t == 0 ? nA : nB;
            if (j >= nt) continue;
            if (!mbar_wait(&bars->p_full[t], j & 1, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
            ODY_FWD_STAMP(blockIdx.x == 0 && blockIdx.y == 0, j, 10 + t * 2);
            if (!have_v) {
              if (!mbar_wait(&bars->v_full[s], ph, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) { ok = false; break; }
              have_v = true;
            }
            tc_fence_after();
            issue_pv(t, j);
            if (j + 1 < nt) {
              if (!have_k1) {
                if (!mbar_wait(&bars->k_full[s1], ph1, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) { ok = false; break; }
                have_k1 = true;
              }
              issue_qk(t, j + 1);      // its commit on s_full[t] also covers the P V just issued
              ODY_FWD_STAMP(blockIdx.x == 0 && blockIdx.y == 0, j, 11 + t * 2);
            } else {
              if (leader) umma_commit(&bars->o_done[t]);
            }
          }
          if (!ok) break;
          if (leader) umma_commit(&bars->v_empty[s]);
          if (have_k1 && leader) umma_commit(&bars->k_empty[s1]);
        }
        if (!ok) {
          if (leader) umma_commit(&bars->drain);
          const long long t0 = clock64();
          while (!mbar_try_wait(&bars->drain, 0) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
        }
      }
    }   // warps 2, 3 idle: they only keep the warpgroups aligned
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (warpgroup t handles tile t)
    // One thread per query row.  The other split that was measured, all eight warps on one tile-block at a time with two
    // threads per row (64 key columns each, partial maxima and sums swapped through shared memory at a 64-thread barrier),
    // was slower: 901 against 1007 TFLOP/s at 8192 tokens x 32 heads, 1030 against 1161 at 32768 x 4, and again with the
    // warp-uniform issue loop, 934 / 1065 against 1085 / 1250.  The exponentials are bound by the special-function unit of
    // each scheduler, which two warps of the same block share, so the block's turn does not get shorter, and the barrier
    // and the halved independent work per thread cost on top.
    reg_inc<PUSH ? REGS_MATH_PUSH : REGS_MATH>();
    const int t = (warp - 4) >> 2;                     // 0 = tile A, 1 = tile B
    const int q = warp & 3;                            // TMEM lane quarter
    const int r = q * 32 + lane;                       // row inside the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const uint32_t col_s = tmem + COL_S + t * BN + lane_off;
    const uint32_t col_o = tmem + COL_O + t * HD + lane_off;
    const int nt = t == 0 ? nA : nB;
    const int qt0 = q0 + t * BM;                       // first query row of this tile
    const int diag = causal ? qt0 / BN : -1;           // block holding this tile's diagonal
    const float sl2 = scale * 1.4426950408889634f;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nt; ++j) {
      const bool tr = blockIdx.x == 0 && blockIdx.y == 0 && (threadIdx.x == 128 || threadIdx.x == 256);
      ODY_FWD_STAMP(tr, j, t * 5 + 0);
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[t], j & 1, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL));
      if (!ok) break;
      ODY_FWD_STAMP(tr, j, t * 5 + 1);
      tc_fence_after();
      uint32_t sv[128];
      tmem_ld_32x32(col_s, sv);
      tmem_ld_32x32(col_s + 32, sv + 32);
      tmem_ld_32x32(col_s + 64, sv + 64);
      tmem_ld_32x32(col_s + 96, sv + 96);
      tmem_ld_wait();
      ODY_FWD_STAMP(tr, j, t * 5 + 2);
      const int kv0 = j * BN;
      if (j == diag) {
#pragma unroll
        for (int c = 0; c < 128; ++c)
          if (c > r) sv[c] = 0xff800000u;               // -inf
      }
      if (kv0 + BN > Tk) {
#pragma unroll
        for (int c = 0; c < 128; ++c)
          if (kv0 + c >= Tk) sv[c] = 0xff800000u;
      }
      // One pass over the 128 scores: exponentials against the maximum in use (packed pairs, x = s * scale * log2(e) - m),
      // P back over S in four 32-column pieces, the row sum, and - on the side, off the dependent chain - the row maximum
      // of THIS block.  The maximum in use only has to be within 2^8 of the true one, so the common case needs no
      // separate maximum pass in front of the exponentials; a block that moves it further is redone (rare).
      const uint64_t sl2_2 = pk2(sl2, sl2);
      float rsum, rmax;
      auto exp_pass = [&]() {
        const uint64_t nm_2 = pk2(-m_used, -m_used);
        uint64_t rs2 = pk2(0.f, 0.f);
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float p0, p1;
            const uint32_t s0 = sv[32 * g + 2 * c], s1 = sv[32 * g + 2 * c + 1];
            mx[c & 1] = fmaxf(mx[c & 1], __uint_as_float(s0));
            mx[2 + (c & 1)] = fmaxf(mx[2 + (c & 1)], __uint_as_float(s1));
            const uint64_t x2 = fma2(pk2u(s0, s1), sl2_2, nm_2);
            upk2(x2, p0, p1);
            p0 = exp2_mufu(p0);
            p1 = exp2_mufu(p1);
            rs2 = add2(rs2, pk2(p0, p1));
            pk[c] = pack_bf16(p0, p1);
          }
          tmem_st_32x16(col_s + g * 16, pk);
        }
        float r0, r1;
        upk2(rs2, r0, r1);
        rsum = r0 + r1;
        rmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      };
      if (j == 0) {
        // first block: there is no maximum in use yet
        float mx[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) mx[i] = __uint_as_float(sv[i]);
#pragma unroll
        for (int c = 4; c < 128; c += 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) mx[i] = fmaxf(mx[i], __uint_as_float(sv[c + i]));
        }
        m_used = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sl2;
        ODY_FWD_STAMP(tr, j, t * 5 + 3);
        exp_pass();
      } else {
        ODY_FWD_STAMP(tr, j, t * 5 + 3);
        exp_pass();
        const float m_new = fmaxf(m_used, rmax * sl2);
        const bool need = (m_new - m_used) > 8.f;
        if (__any_sync(0xffffffffu, need)) {
          // the running maximum moved by more than 2^8 for some row of this warp: rescale O and l, redo the block.
          // P V of block j-1 completed before S(j) was announced and P V of block j waits for this thread, so O is ours.
          const float alpha = need ? exp2_mufu(m_used - m_new) : 1.f;
          if (need) m_used = m_new;
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t o[16];
            tmem_ld_32x16(col_o + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(col_o + c * 16, o);
          }
          exp_pass();
        }
      }
      l += rsum;
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->p_full[t]);
      ODY_FWD_STAMP(tr, j, t * 5 + 4);
    }
    // epilogue: O / l -> bf16 -> swizzled smem (this tile's Q is dead by now) -> TMA store; lse
    if (ok && nt > 0) ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_done[t], 0, abort_flag, err, ODY_ERR_TIMEOUT_MISC));
    uint8_t* stage = sQ + t * TILE_BYTES;
    if (ok && nt > 0) {
      tc_fence_after();
      const float inv_l = 1.f / l;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(col_o + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 v4;
          v4.x = pack_bf16(__uint_as_float(o[8 * i + 0]) * inv_l, __uint_as_float(o[8 * i + 1]) * inv_l);
          v4.y = pack_bf16(__uint_as_float(o[8 * i + 2]) * inv_l, __uint_as_float(o[8 * i + 3]) * inv_l);
          v4.z = pack_bf16(__uint_as_float(o[8 * i + 4]) * inv_l, __uint_as_float(o[8 * i + 5]) * inv_l);
          v4.w = pack_bf16(__uint_as_float(o[8 * i + 6]) * inv_l, __uint_as_float(o[8 * i + 7]) * inv_l);
          const int chunk = (c & 1) * 4 + i;            // 16-byte chunk inside the 128-byte row of half c / 2
          *reinterpret_cast<uint4*>(stage + (c >> 1) * HALF_BYTES + r * 128 + ((chunk ^ (r & 7)) << 4)) = v4;
        }
      }
      if (qt0 + r < Tq) lse[(int64_t)head * Tq + qt0 + r] = (m_used + log2f(l)) * 0.6931471805599453f;
      fence_proxy_async_smem();
    }
    tc_fence_before();
    const bool all_ok = named_barrier_and(1 + t, 128, ok);
    if (all_ok && nt > 0 && q == 0 && lane == 0 && !*abort_flag) {
      tma_store_3d(&tmO, stage, 0, head, qt0);
      tma_store_3d(&tmO, stage + HALF_BYTES, 64, head, qt0);
      if (osplit.rows > 0) {
        const int d = qt0 / osplit.rows;
        tma_store_3d(&osplit.m[d], stage, 0, head, qt0 - d * osplit.rows);
        tma_store_3d(&osplit.m[d], stage + HALF_BYTES, 64, head, qt0 - d * osplit.rows);
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

// q/k/v/o: bf16, head_dim 128, element strides: *_row (token pitch), heads packed (pitch 128).
extern "C" int ody_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int Tq, int Tk, int H,
                             int Hkv, int64_t q_row, int64_t k_row, int64_t v_row, int64_t o_row, int causal,
                             float scale, int* err, cudaStream_t st) {
  return ody_flash_fwd_ex(q, k, v, o, lse, Tq, Tk, H, Hkv, q_row, k_row, v_row, o_row, causal, scale, nullptr, nullptr, 0, 0, 0,
                          err, st);
}

// CTAs of the forward grid for Tq query rows and H heads: what a push description's n_cta may not exceed.
extern "C" int ody_flash_fwd_ctas(int Tq, int H) {
  return ((Tq + ody::fwd::CTA_ROWS - 1) / ody::fwd::CTA_ROWS) * H;
}

#ifdef ODY_ATTN_TRACE
extern "C" int ody_flash_fwd_set_trace(long long* buf) { return (int)cudaMemcpyToSymbol(g_fwd_trace_buf, &buf, sizeof(buf)); }
#else
extern "C" int ody_flash_fwd_set_trace(long long*) { return (int)cudaErrorNotSupported; }
#endif

static int g_fwd_ks32 = 0;
// 1: Q and K tiles as eight 32-byte-swizzled slices (KS32 above), 0: as two 128-byte-swizzled halves
extern "C" int ody_flash_fwd_set_kslice(int on) {
  g_fwd_ks32 = on ? 1 : 0;
  return 0;
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
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_fwd_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_fwd_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_fwd_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap tQ, tK, tV, tO;
  int r;
  const bool ks32 = g_fwd_ks32 != 0;
  if ((r = make_tmap_3d_bf16(&tQ, q, HD, H, Tq, HD * 2, q_row * 2, ks32 ? 16 : 64, 1, BM, ks32))) return 730000 + r;
  if ((r = make_tmap_3d_bf16(&tK, k, HD, Hkv, Tk, HD * 2, k_row * 2, ks32 ? 16 : 64, 1, BN, ks32))) return 740000 + r;
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
  dim3 grid((Tq + CTA_ROWS - 1) / CTA_ROWS, H);
  gc::GatherParams pp;
  memset(&pp, 0, sizeof(pp));
  if (push != nullptr) {
    if ((r = gc::fill_gather(pp, push))) return r;
    const int ctas = (int)(grid.x * grid.y);
    if (push->n_cta <= 0 || push->n_cta > ctas) return (int)cudaErrorInvalidValue;
    if (ks32)
      flash_fwd_kernel<true, true><<<grid, NUM_THREADS_PUSH, SMEM_TOTAL, st>>>(tQ, tK, tV, tO, lse, Tq, Tk, H, Hkv, causal, scale, err, pp, push->n_cta, sm);
    else
      flash_fwd_kernel<true, false><<<grid, NUM_THREADS_PUSH, SMEM_TOTAL, st>>>(tQ, tK, tV, tO, lse, Tq, Tk, H, Hkv, causal, scale, err, pp, push->n_cta, sm);
  } else if (ks32) {
    flash_fwd_kernel<false, true><<<grid, NUM_THREADS, SMEM_TOTAL, st>>>(tQ, tK, tV, tO, lse, Tq, Tk, H, Hkv, causal, scale, err, pp, 0, sm);
  } else {
    flash_fwd_kernel<false, false><<<grid, NUM_THREADS, SMEM_TOTAL, st>>>(tQ, tK, tV, tO, lse, Tq, Tk, H, Hkv, causal, scale, err, pp, 0, sm);
  }
  return (int)cudaGetLastError();
}
