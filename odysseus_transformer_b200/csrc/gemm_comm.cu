// GEMM fused with its collective over NVLink peer memory (sm_100a): ONE kernel does the transfer and
// the tcgen05 math, tile by tile.
//
//   GATHER (all-gather -> GEMM): one operand is the row-wise concatenation of every rank's shard.  Every
//     CTA carries four extra "comm" warps that PUSH this rank's shard into all ranks' gathered buffers
//     with plain 16-byte peer stores (NVLink traffic spread over all SMs: one SM sustains only a few GB/s
//     of remote traffic, 148 of them saturate the links), raising a counter per row block at the
//     destination; the producer thread of each GEMM CTA waits for the counters of the rows an operand
//     tile needs before it issues that tile's TMA load from the local gathered buffer.  Tile (or
//     k-block) order is rotated so each rank starts on its own shard.  Serves the sequence all-gather
//     of the column-parallel linears (reference utils/linear_tpsp.py:159-173,205-217) and the weight
//     all-gather of the ZeRO-3 linears (reference utils/linear_zero3.py:35-44,62-68).
//   SCATTER (GEMM -> reduce-scatter): the epilogue pushes every output row straight from registers into
//     the staging slot of the rank that owns it (plain peer stores); tiles owned by other ranks are
//     computed first.  When its tiles are done each CTA reduces part of this rank's own rows over the N
//     staging slots in fp32 as soon as every source has signalled.  Serves the row-parallel output
//     reduce-scatter, the dgrad reduce-scatter and the ZeRO-3 wgrad reduce-scatter
//     (reference utils/linear_tpsp.py:35-58,247-256; utils/linear_zero3.py:76-84).
//
// Cross-GPU ordering uses monotonically increasing epoch words in symmetric memory (ready / done /
// arrived / consumed), written with release.sys and polled with acquire.sys.  Every poll is bounded and
// reports through the status word; nothing here can spin forever.
#include "ody_kernels.h"

// Every wait in this file can depend on a peer (the pipeline stalls while rows are in flight), so the
// pipeline's own barrier waits get twice the run-time peer limit instead of the 1 s of the single-GPU
// kernels: a peer that never delivers is then reported as such (the peer wait gives up first and raises
// the abort flag that ends the others).  ody_set_peer_wait_limit changes the limit for the current device.
#define ODY_SPIN_LIMIT_CYCLES (2 * ody::gc::g_peer_spin_limit)
#include "peer_comm.cuh"

namespace ody {
namespace gc {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_COLS = 64, EPI_BYTES = BM * EPI_COLS * 2;
constexpr int SMEM_TILES = STAGES * STAGE_BYTES + 2 * EPI_BYTES;
constexpr int SMEM_TOTAL = SMEM_TILES + 512 + 1024;
constexpr int NUM_THREADS = 192;          // TMA warp, MMA warp, 4 epilogue warps
constexpr int GROUP_M = 16;

struct ScatterParams {
  __nv_bfloat16* stage_peer[MAX_RANKS];   // owner p's staging: [n_ranks (source)][chunk_rows][ldc]
  uint32_t* arrived_peer[MAX_RANKS];      // arrived_peer[p][rank] += 1 per tile pushed to owner p
  uint32_t* consumed_peer[MAX_RANKS];     // consumed_peer[p][rank] <- epoch : "owner `rank` has reduced this slot"
  uint32_t* arrived_local;                // [n_ranks] counters written by sources
  uint32_t* consumed_local;               // [n_ranks] epochs written by owners
  uint32_t* reduce_counter;               // local: CTAs that finished their part of the reduction
  __nv_bfloat16* out;                     // [chunk_rows, N] result rows of this rank
  int64_t out_ld;
  int n_ranks, rank, chunk_rows;
  uint32_t epoch, prev_epoch;
  uint32_t arrived_target;                // cumulative: GEMM CTAs of each source * uses
  uint32_t reduce_target;                 // cumulative: n_gemm CTAs * uses
  // SCATTER == 2 (all-to-all on columns): columns [o * a2a_cols, (o + 1) * a2a_cols) of row r go to rank o's buffer
  // stage_peer[o] at row a2a_row0 + r, column a2a_col0 + (c - o * a2a_cols), row pitch a2a_ld
  int a2a_cols;
  int64_t a2a_ld, a2a_row0, a2a_col0;
  unsigned long long* wait_acc;           // optional running totals (ns): [1] += the time owners waited for the sources' tiles
  const __nv_bfloat16* residual;          // optional, added to the result: SCATTER == 1 [chunk_rows, N], this rank's reduced
                                          // rows; SCATTER == 0 [M, N]
  int64_t residual_ld;
};

struct Bars {
  uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], drain;
  uint32_t tmem_base;
  int abort_flag;
  uint32_t seen[64];            // bitset of gathered row blocks this CTA has already found complete
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int shift_m, int shift_n, int& tm, int& tn) {
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsize = min(GROUP_M, tiles_m - first_m);
  const int local = tile - g * per_group;
  tm = first_m + local % gsize;
  tn = local / gsize;
  tm += shift_m; if (tm >= tiles_m) tm -= tiles_m;
  tn += shift_n; if (tn >= tiles_n) tn -= tiles_n;
}

__device__ __forceinline__ bool epi_all_ok(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 2, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(r) : "r"((uint32_t)ok) : "memory");
  return r != 0;
}

// Wait until the gathered rows [row0, row0 + nrows) have landed in the local gathered buffer.  Once every
// copy CTA has reported a whole shard done (cta_counters) that shard is remembered in `done_mask` and costs
// no further polling - with a K-gathered operand every k-block would otherwise pay a flag read.
__device__ __forceinline__ bool wait_rows(const GatherParams& g, int row0, int nrows, int& last_ok, uint32_t& done_mask,
                                          uint32_t& ctr_checked, uint32_t* seen, int lookahead, volatile int* abort_flag, int* err) {
  const int total_rows = g.n_ranks * g.chunk_rows;
  const int UR = g.unit_rows;
  const int nb = g.chunk_rows / UR;
  const int rend = min(row0 + nrows, total_rows);
  bool waited = false;
  for (int row = row0; row < rend;) {
    const int p = row / g.chunk_rows;
    if ((done_mask >> p) & 1u) { row = (p + 1) * g.chunk_rows; continue; }
    const int ric = row - p * g.chunk_rows;
    const int blk = ric / UR;
    const int idx = p * nb + blk;
    const bool cacheable = idx < 64 * 32;
    if (idx != last_ok && !(cacheable && ((seen[idx >> 5] >> (idx & 31)) & 1u))) {
      if (!((ctr_checked >> p) & 1u)) {          // whole-shard counter: looked at once per tile and shard
        ctr_checked |= 1u << p;
        if ((int32_t)(ld_acquire_sys(g.counters_local + p) - g.counter_target) >= 0) {
          done_mask |= 1u << p;
          waited = true;
          row = (p + 1) * g.chunk_rows;
          continue;
        }
      }
      // `lookahead` > 1 (K-gathered operands, where every tile walks all rows in order) waits for a run of
      // row blocks at once so the proxy fence below - several microseconds - is paid once per run
      const int run = min(lookahead, nb - blk);
      for (int j = 0; j < run; ++j) {
        const int id = idx + j;
        if (id < 64 * 32 && ((seen[id >> 5] >> (id & 31)) & 1u)) continue;
        if (!wait_word<true>(g.flags_local + id, g.flag_target, abort_flag, err, ODY_ERR_TIMEOUT_PEER)) return false;
        if (id < 64 * 32) seen[id >> 5] |= 1u << (id & 31);
      }
      last_ok = idx;
      waited = true;
    }
    row = p * g.chunk_rows + (blk + 1) * UR;
  }
  if (waited) fence_proxy_async_all();   // the data was written through the async proxy by another CTA
  return true;
}

// Push-only launch: starts a chain of prefetching GEMMs (the first weight of a pass has no earlier GEMM
// to ride on).
__global__ void __launch_bounds__(COMM_THREADS) push_shard_kernel(const __grid_constant__ GatherParams pp, int* __restrict__ err) {
  __shared__ int abort_flag;
  if (threadIdx.x == 0) abort_flag = 0;
  __syncthreads();
  comm_warps_main(pp, (int)blockIdx.x, (int)gridDim.x, 0, &abort_flag, err);
}

// ------------------------------------------------------------------------------------------- kernel
// GATHER: 0 none, 1 operand A is gathered, 2 operand B is gathered.  SCATTER: 0 plain TMA-store epilogue,
// 1 push rows to their owner and reduce own rows, 2 all-to-all: push column groups to their owner (the
// Ulysses sequence<->head exchange, yunchang SeqAllToAll4D called at reference decoder/ulysses.py:40-47;
// the receivers wait on the per-source counters with ody_wait_flags).
// ROPE: the epilogue rotates the q / k heads of a packed projection (RopeEpi, sm100.cuh); compiled only where a
// q|k|v projection can be the product, so that the other instances keep their register allocation.
template <int LAYOUT, int GATHER, int SCATTER, bool ROPE>
__global__ void __launch_bounds__(NUM_THREADS + COMM_THREADS, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ GatherParams gp,
                 const __grid_constant__ GatherParams pp, const __grid_constant__ ScatterParams sp, int M, int N, int K, int64_t ldc, int n_gemm,
                 int mn3d, const RopeEpi rp, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Bars* bars = (Bars*)(smem + SMEM_TILES);
  uint8_t* epi = smem + STAGES * STAGE_BYTES;
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gemm_idx = (int)blockIdx.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&bars->tmem_full[b], 1); mbar_init(&bars->tmem_empty[b], 128); }
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    for (int i = 0; i < 64; ++i) bars->seen[i] = 0;
    mbar_fence_init();
  }

  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (K + BK - 1) / BK;
  constexpr bool A_MN = (LAYOUT == 2), B_MN = (LAYOUT != 0);
  constexpr uint32_t IDESC = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
  // which GEMM dimension the gathered operand's memory rows run along
  constexpr bool G_ROWS_M = (GATHER == 1 && LAYOUT != 2);
  constexpr bool G_ROWS_N = (GATHER == 2 && LAYOUT == 0);
  constexpr bool G_ROWS_K = (GATHER == 1 && LAYOUT == 2) || (GATHER == 2 && LAYOUT != 0);
  int shift_m = 0, shift_n = 0, shift_k = 0;
  if (G_ROWS_M) shift_m = (int)(((int64_t)gp.rank * gp.chunk_rows) / BM) % tiles_m;
  if (G_ROWS_N) shift_n = (int)(((int64_t)gp.rank * gp.chunk_rows) / BN) % tiles_n;
  if (G_ROWS_K) shift_k = (int)(((int64_t)gp.rank * gp.chunk_rows) / BK) % kblocks;
  if (SCATTER == 1) shift_m = (int)((((int64_t)(sp.rank + 1) * sp.chunk_rows + BM - 1) / BM) % tiles_m);   // others' rows first

  if (warp == 1) { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (GATHER && warp >= NUM_THREADS / 32) {
    // gp describes the operand this GEMM consumes, pp the shard these warps push: the same slot, or the
    // NEXT linear's weight (prefetch), so that its all-gather hides behind this GEMM's math
    comm_warps_main(pp, gemm_idx, n_gemm, NUM_THREADS, abort_flag, err);
  } else if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; int issued = 0; bool ok = true; int last_ok = -1; uint32_t done_mask = 0, ctr_checked = 0;
      unsigned long long waited_ns = 0;
      const bool timed = GATHER && (gp.stats != nullptr || gp.wait_acc != nullptr);
      const uint32_t all_ranks_mask = GATHER ? ((1u << gp.n_ranks) - 1u) : 0u;
      for (int tile = gemm_idx; tile < num_tiles && ok; tile += n_gemm) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, shift_m, shift_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        ctr_checked = 0;
        if (G_ROWS_K && done_mask != all_ranks_mask) {
          // once per tile: shards whose every pusher has reported need no per-k-block bookkeeping at all
          for (int p = 0; p < gp.n_ranks; ++p)
            if (!((done_mask >> p) & 1u) && (int32_t)(ld_acquire_sys(gp.counters_local + p) - gp.counter_target) >= 0)
              done_mask |= 1u << p;
          if (done_mask == all_ranks_mask) fence_proxy_async_all();
        }
        if (G_ROWS_M || G_ROWS_N) {
          const unsigned long long t0 = (GATHER && timed) ? global_ns() : 0;
          if (G_ROWS_M && !wait_rows(gp, m0, BM, last_ok, done_mask, ctr_checked, bars->seen, 1, abort_flag, err)) { ok = false; break; }
          if (G_ROWS_N && !wait_rows(gp, n0, BN, last_ok, done_mask, ctr_checked, bars->seen, 1, abort_flag, err)) { ok = false; break; }
          if (GATHER && timed) waited_ns += global_ns() - t0;
        }
        for (int kb = 0; kb < kblocks; ++kb) {
          int kbr = kb + shift_k; if (kbr >= kblocks) kbr -= kblocks;
          const int k0 = kbr * BK;
          if (G_ROWS_K && done_mask != all_ranks_mask) {
            const unsigned long long t0 = timed ? global_ns() : 0;
            if (!wait_rows(gp, k0, BK, last_ok, done_mask, ctr_checked, bars->seen, 16, abort_flag, err)) { ok = false; break; }
            if (timed) waited_ns += global_ns() - t0;
          }
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          mbar_expect_tx(&bars->full[stage], STAGE_BYTES);
          if (!A_MN) tma_load_2d(sA, &tmA, k0, m0, &bars->full[stage]);
          else if (mn3d & 1) tma_load_3d(sA, &tmA, 0, k0, m0 / 64, &bars->full[stage]);
          else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sA + j * 8192, &tmA, m0 + 64 * j, k0, &bars->full[stage]);
          }
          if (!B_MN) tma_load_2d(sB, &tmB, k0, n0, &bars->full[stage]);
          else if (mn3d & 2) tma_load_3d(sB, &tmB, 0, k0, n0 / 64, &bars->full[stage]);
          else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sB + j * 8192, &tmB, n0 + 64 * j, k0, &bars->full[stage]);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (GATHER && gp.stats) gp.stats[gemm_idx * 4 + 2] = waited_ns;
      if (GATHER && gp.wait_acc != nullptr && waited_ns) atomicAdd(gp.wait_acc, waited_ns);
      if (!ok || *abort_flag) {
        int n = issued < STAGES ? issued : STAGES;
        for (int i = 0; i < n; ++i) {
          if (--stage < 0) { stage = STAGES - 1; phase ^= 1; }
          const long long t0 = clock64();
          while (!mbar_try_wait(&bars->full[stage], phase) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
        }
      }
    }
  } else if (warp == 1) {
    {
      // every lane runs the control flow, so the compiler keeps descriptors and loop state in uniform registers and an MMA
      // costs a few instructions; one elected lane issues the tcgen05 instructions (benchmarks/mma_issue_rate.cu)
      const bool leader = elect_one();
      int stage = 0; uint32_t phase = 0; int local_tile = 0; bool ok = true;
      const uint32_t s0 = smem_u32(smem);
      const uint64_t adesc0 = A_MN ? make_smem_desc(s0, 8192, 1024) : make_smem_desc(s0, 16, 1024);
      const uint64_t bdesc0 = B_MN ? make_smem_desc(s0 + A_BYTES, 8192, 1024) : make_smem_desc(s0 + A_BYTES, 16, 1024);
      for (int tile = gemm_idx; tile < num_tiles && ok; tile += n_gemm, ++local_tile) {
        const int buf = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[buf], acc_phase ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint64_t a0 = desc_advance(adesc0, stage * STAGE_BYTES), b0 = desc_advance(bdesc0, stage * STAGE_BYTES);
          if (leader) umma_ss(d_tmem, a0, b0, IDESC, kb > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < BK / UMMA_K; ++kk)
            if (leader) umma_ss(d_tmem, desc_advance(a0, kk * (A_MN ? 2048 : 32)), desc_advance(b0, kk * (B_MN ? 2048 : 32)), IDESC, 1u);
          if (leader) umma_commit(&bars->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok && leader) umma_commit(&bars->tmem_full[buf]);
      }
      if (!ok || *abort_flag) {
        if (leader) umma_commit(&bars->drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(&bars->drain, 0) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int et = threadIdx.x - 64;                 // 0..127 among the epilogue threads
    const bool store_thread = (et == 0);
    int local_tile = 0;
    uint32_t verified = 0;                            // owners whose staging slot is known to be free
    bool alive = true;
    int remaining[MAX_RANKS];                         // tiles this CTA still has to push to each owner (store_thread only)
    if (SCATTER == 1 && store_thread) {
#pragma unroll
      for (int o = 0; o < MAX_RANKS; ++o) remaining[o] = 0;
      for (int tile = gemm_idx; tile < num_tiles; tile += n_gemm) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, shift_m, shift_n, tm, tn);
        const int last_row = min(tm * BM + BM, M) - 1;
        const int o0 = min(tm * BM / sp.chunk_rows, sp.n_ranks - 1), o1 = min(last_row / sp.chunk_rows, sp.n_ranks - 1);
#pragma unroll
        for (int o = 0; o < MAX_RANKS; ++o) if (o >= o0 && o <= o1) ++remaining[o];
      }
      // owners this CTA never writes to hear from it right away
#pragma unroll
      for (int o = 0; o < MAX_RANKS; ++o)
        if (o < sp.n_ranks && remaining[o] == 0) red_release_sys_add(sp.arrived_peer[o] + sp.rank, 1);
    }
    for (int tile = gemm_idx; tile < num_tiles; tile += n_gemm, ++local_tile) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, shift_m, shift_n, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      const int buf = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      bool ok = mbar_wait(&bars->tmem_full[buf], acc_phase, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL);
      // rows this thread pushes in the coalesced copy phase: (et / 8) + 16 * i, 16-byte chunk et % 8
      __nv_bfloat16* push_rows[8];
      if (SCATTER == 2) {
        // every destination must have consumed what its buffer held before (checked once per CTA)
        if (verified == 0 && et < sp.n_ranks && et != sp.rank)
          ok = wait_word<true>(sp.consumed_local + et, sp.prev_epoch, abort_flag, err, ODY_ERR_TIMEOUT_PEER) && ok;
        verified = 1;
      }
      if (SCATTER == 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = m0 + (et >> 3) + 16 * i;
          push_rows[i] = nullptr;
          if (row < M) {
            const int owner = min(row / sp.chunk_rows, sp.n_ranks - 1);
            if (ok && !((verified >> owner) & 1u)) {
              // the owner must have reduced what this slot held before it is overwritten
              ok = wait_word<true>(sp.consumed_local + owner, sp.prev_epoch, abort_flag, err, ODY_ERR_TIMEOUT_PEER);
              verified |= 1u << owner;
            }
            push_rows[i] = sp.stage_peer[owner] + ((int64_t)sp.rank * sp.chunk_rows + (row - owner * sp.chunk_rows)) * ldc;
          }
        }
      }
      if (!epi_all_ok(ok)) { alive = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < BN / EPI_COLS; ++c) {
        uint8_t* sbuf = epi + (c & 1) * EPI_BYTES;
        if (!SCATTER) {
          if (store_thread) tma_store_wait_read<1>();
          named_barrier(1, 128);
        }
        const uint32_t taddr = tmem_base + buf * BN + c * EPI_COLS + ((uint32_t)(q * 32) << 16);
        uint32_t v[64];
        tmem_ld_32x32(taddr, v);
        tmem_ld_32x32(taddr + 32, v + 32);
        tmem_ld_wait();
        const int col0 = n0 + c * EPI_COLS;
        if (ROPE && SCATTER != 1 && rope_epi_wants(rp, col0)) {
          // rotary embedding of a q / k head: the other half of the head is still in the accumulator
          uint32_t w[64];
          const uint32_t paddr = (c & 1) ? taddr - EPI_COLS : taddr + EPI_COLS;
          tmem_ld_32x32(paddr, w);
          tmem_ld_32x32(paddr + 32, w + 32);
          tmem_ld_wait();
          if (m0 + r < M) rope_epi_apply(rp, m0 + r, c & 1, v, w);
        }
        if (c == BN / EPI_COLS - 1) { tc_fence_before(); mbar_arrive(&bars->tmem_empty[buf]); }
        if (SCATTER) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 pk;
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int t = 0; t < 4; ++t)
              p2[t] = __floats2bfloat162_rn(__uint_as_float(v[j * 8 + 2 * t]), __uint_as_float(v[j * 8 + 2 * t + 1]));
            *reinterpret_cast<uint4*>(sbuf + r * 128 + ((j ^ (r & 7)) << 4)) = pk;
          }
          named_barrier(1, 128);
          // 8 consecutive threads write one 128-byte row segment: full lines on the wire
          const int j = et & 7;
          if (SCATTER == 2) {
            if (col0 < N) {
              const int owner = col0 / sp.a2a_cols;
              __nv_bfloat16* base = sp.stage_peer[owner] + sp.a2a_col0 + (col0 - owner * sp.a2a_cols) + j * 8;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rr = (et >> 3) + 16 * i;
                if (m0 + rr < M)
                  *reinterpret_cast<uint4*>(base + (sp.a2a_row0 + m0 + rr) * sp.a2a_ld) =
                      *reinterpret_cast<const uint4*>(sbuf + rr * 128 + ((j ^ (rr & 7)) << 4));
              }
            }
          } else if (col0 + j * 8 < N) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = (et >> 3) + 16 * i;
              if (push_rows[i] != nullptr)
                *reinterpret_cast<uint4*>(push_rows[i] + col0 + j * 8) =
                    *reinterpret_cast<const uint4*>(sbuf + rr * 128 + ((j ^ (rr & 7)) << 4));
            }
          }
        } else {
          if (sp.residual != nullptr && m0 + r < M) {
            // the residual stream's row joins the product before it is rounded
            const __nv_bfloat16* cp = sp.residual + (int64_t)(m0 + r) * sp.residual_ld + col0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (col0 + j * 8 < N) {   // N is a multiple of 8
                const uint4 old = *reinterpret_cast<const uint4*>(cp + j * 8);
                const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                  const float2 f = __bfloat1622float2(o2[t]);
                  v[j * 8 + 2 * t] = __float_as_uint(__uint_as_float(v[j * 8 + 2 * t]) + f.x);
                  v[j * 8 + 2 * t + 1] = __float_as_uint(__uint_as_float(v[j * 8 + 2 * t + 1]) + f.y);
                }
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 pk;
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int t = 0; t < 4; ++t)
              p2[t] = __floats2bfloat162_rn(__uint_as_float(v[j * 8 + 2 * t]), __uint_as_float(v[j * 8 + 2 * t + 1]));
            *reinterpret_cast<uint4*>(sbuf + r * 128 + ((j ^ (r & 7)) << 4)) = pk;
          }
          fence_proxy_async_smem();
          named_barrier(1, 128);
          if (store_thread && col0 < N) { tma_store_2d(&tmC, sbuf, col0, m0); tma_store_commit(); }
        }
      }
      if (SCATTER == 1) {
        // Every row of this tile is on its way.  When it was this CTA's last tile for an owner, one thread
        // fences at system scope (the barrier makes the other threads' stores part of what it releases) and
        // tells that owner that this CTA is done with it.
        named_barrier(1, 128);
        if (store_thread) {
          const int last_row = min(m0 + BM, M) - 1;
          const int o0 = min(m0 / sp.chunk_rows, sp.n_ranks - 1), o1 = min(last_row / sp.chunk_rows, sp.n_ranks - 1);
          bool fenced = false;
#pragma unroll
          for (int o = 0; o < MAX_RANKS; ++o) {
            if (o >= o0 && o <= o1 && --remaining[o] == 0) {
              if (!fenced) { __threadfence_system(); fenced = true; }
              red_release_sys_add(sp.arrived_peer[o] + sp.rank, 1);
            }
          }
        }
      }
    }
    if (!SCATTER) {
      if (store_thread) tma_store_wait<0>();
    } else if (SCATTER == 2) {
      // all of this CTA's column groups are on their way: one fence, then tell every destination
      named_barrier(1, 128);
      if (store_thread && alive) {
        __threadfence_system();
        for (int o = 0; o < sp.n_ranks; ++o) red_release_sys_add(sp.arrived_peer[o] + sp.rank, 1);
      }
    } else if (alive) {
      // reduce this rank's rows over the N source slots once every source has delivered all its tiles
      bool ok = true;
      const unsigned long long tw0 = (sp.wait_acc != nullptr && et == 0) ? global_ns() : 0;
      if (et < sp.n_ranks) ok = wait_word<true>(sp.arrived_local + et, sp.arrived_target, abort_flag, err, ODY_ERR_TIMEOUT_PEER);
      const bool all_ok = epi_all_ok(ok);
      if (sp.wait_acc != nullptr && et == 0) atomicAdd(sp.wait_acc + 1, global_ns() - tw0);
      if (all_ok) {
        const __nv_bfloat16* mine = sp.stage_peer[sp.rank];
        const int vec_per_row = N / 8;
        const int64_t total = (int64_t)sp.chunk_rows * vec_per_row;
        const int64_t slot = (int64_t)sp.chunk_rows * ldc;
        const int64_t stride = (int64_t)n_gemm * 128;
        constexpr int RU = 8;
        for (int64_t i0 = (int64_t)gemm_idx * 128 + et; i0 < total; i0 += RU * stride) {
          float acc[RU][8];
          int64_t off[RU];
          bool live[RU];
#pragma unroll
          for (int u = 0; u < RU; ++u) {
            const int64_t i = i0 + u * stride;
            live[u] = i < total;
            const int64_t rr = live[u] ? i / vec_per_row : 0;
            const int cc = live[u] ? (int)(i % vec_per_row) * 8 : 0;
            off[u] = rr * ldc + cc;
#pragma unroll
            for (int t = 0; t < 8; ++t) acc[u][t] = 0.f;
            if (sp.residual != nullptr && live[u]) {
              // the residual stream's rows of this rank start the sum
              const uint4 pk = *reinterpret_cast<const uint4*>(sp.residual + rr * sp.residual_ld + cc);
              const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                const float2 f = __bfloat1622float2(p2[t]);
                acc[u][2 * t] = f.x;
                acc[u][2 * t + 1] = f.y;
              }
            }
          }
          for (int s = 0; s < sp.n_ranks; ++s) {
            uint4 pk[RU];
#pragma unroll
            for (int u = 0; u < RU; ++u)
              pk[u] = live[u] ? *reinterpret_cast<const uint4*>(mine + s * slot + off[u]) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < RU; ++u) {
              const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&pk[u]);
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                const float2 f = __bfloat1622float2(p2[t]);
                acc[u][2 * t] += f.x;
                acc[u][2 * t + 1] += f.y;
              }
            }
          }
#pragma unroll
          for (int u = 0; u < RU; ++u) {
            if (!live[u]) continue;
            const int64_t i = i0 + u * stride;
            const int64_t rr = i / vec_per_row;
            const int cc = (int)(i % vec_per_row) * 8;
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int t = 0; t < 4; ++t) o2[t] = __floats2bfloat162_rn(acc[u][2 * t], acc[u][2 * t + 1]);
            *reinterpret_cast<uint4*>(sp.out + rr * sp.out_ld + cc) = o;
          }
        }
        __threadfence();
        named_barrier(1, 128);
        if (store_thread && atomicAdd(sp.reduce_counter, 1) + 1 == sp.reduce_target) {
          for (int s = 0; s < sp.n_ranks; ++s) st_release_sys(sp.consumed_peer[s] + sp.rank, sp.epoch);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
  if (GATHER && threadIdx.x == 0 && gp.stats != nullptr) gp.stats[gemm_idx * 4 + 3] = global_ns();
  if (GATHER && threadIdx.x == 0) {
    // the last GEMM CTA to finish tells every pusher that this rank's gathered buffer may be overwritten
    __threadfence();
    if (atomicAdd(gp.gemm_done, 1) + 1 == gp.gemm_done_target) {
      __threadfence_system();
      for (int s = 1; s < gp.n_ranks; ++s) {
        const int p = (gp.rank + s) % gp.n_ranks;
        st_release_sys(gp.free_peer[p] + gp.rank, gp.epoch);
      }
    }
  }
}

}  // namespace gc
}  // namespace ody

namespace ody {
namespace gc {

static int g_sms = 0;
// per-device running totals of time spent waiting on other GPUs (ody_set_wait_accumulator); null = not collected
static unsigned long long* g_wait_acc[64] = {nullptr};
static unsigned long long* wait_acc_here() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  return g_wait_acc[dev];
}

template <int LAYOUT, int GATHER, int SCATTER, bool ROPE>
static int launch(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                  const OdyGatherDesc* gd, const OdyGatherDesc* pd, const OdyScatterDesc* sd, const OdyEpilogue* epi, int* err,
                  cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_comm_kernel<LAYOUT, GATHER, SCATTER, ROPE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (g_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap tA, tB, tC;
  int r;
  int mn3d = 0;   // bit 0: A tile is one blocked 3-D TMA load, bit 1: B tile is
  if (LAYOUT == 2 && (M % 64) == 0) { r = make_tmap_mn_blocked_bf16(&tA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, BK, BM / 64); mn3d |= 1; }
  else if (LAYOUT == 2) r = make_tmap_2d_bf16(&tA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, 64);
  else r = make_tmap_2d_bf16(&tA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, 64, BM);
  if (r) return 700000 + r;
  if (LAYOUT == 0) r = make_tmap_2d_bf16(&tB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, 64, BN);
  else if ((N % 64) == 0) { r = make_tmap_mn_blocked_bf16(&tB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, BK, BN / 64); mn3d |= 2; }
  else r = make_tmap_2d_bf16(&tB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, 64);
  if (r) return 710000 + r;
  GatherParams gp;
  ScatterParams sp;
  memset(&gp, 0, sizeof(gp));
  memset(&sp, 0, sizeof(sp));
  GatherParams pp;
  memset(&pp, 0, sizeof(pp));
  bool has_push = false;
  if (GATHER) {
    if ((r = fill_gather(gp, gd))) return r;
    gp.wait_acc = wait_acc_here();
    if (pd != nullptr) {
      if ((r = fill_gather(pp, pd))) return r;
      if (pd->shard == nullptr || (pd->shard_ld % 8) || ((uintptr_t)pd->shard & 15)) return (int)cudaErrorInvalidValue;
      has_push = true;
    }
  }
  if (SCATTER) {
    if (sd == nullptr || sd->n_ranks < 2 || sd->n_ranks > MAX_RANKS) return (int)cudaErrorInvalidValue;
    if (SCATTER == 1 && sd->chunk_rows * sd->n_ranks != M) return (int)cudaErrorInvalidValue;
    if (SCATTER == 2 && (sd->a2a_cols <= 0 || (sd->a2a_cols % 64) || (int64_t)sd->a2a_cols * sd->n_ranks != N || (sd->a2a_ld % 8) ||
                         (sd->a2a_col0 % 8) || sd->a2a_row0 < 0))
      return (int)cudaErrorInvalidValue;
    sp.a2a_cols = sd->a2a_cols; sp.a2a_ld = sd->a2a_ld; sp.a2a_row0 = sd->a2a_row0; sp.a2a_col0 = sd->a2a_col0;
    for (int p = 0; p < sd->n_ranks; ++p) {
      sp.stage_peer[p] = (__nv_bfloat16*)sd->stage_peer[p];
      sp.arrived_peer[p] = sd->arrived_peer[p];
      sp.consumed_peer[p] = sd->consumed_peer[p];
    }
    sp.arrived_local = sd->arrived_peer[sd->rank];
    sp.consumed_local = sd->consumed_peer[sd->rank];
    sp.reduce_counter = sd->reduce_counter;
    sp.out = (__nv_bfloat16*)sd->out;
    sp.out_ld = sd->out_ld;
    sp.n_ranks = sd->n_ranks; sp.rank = sd->rank; sp.chunk_rows = sd->chunk_rows;
    sp.epoch = sd->epoch; sp.prev_epoch = sd->prev_epoch;
    sp.wait_acc = wait_acc_here();
    // C is only a placeholder for the tensor map in this mode: staging is dense with ld = N
    ldc = N;
    C = sd->stage_peer[sd->rank];
  }
  RopeEpi rp;
  rp.cos = rp.sin = nullptr;
  rp.period_cols = rp.rot_cols = 0;
  if (epi != nullptr) {
    // the residual joins the reduction of a reduce-scatter or the plain epilogue, the rotation the epilogues that keep whole rows
    if (epi->residual != nullptr) {
      if (SCATTER == 2 || (epi->residual_ld % 8) || ((uintptr_t)epi->residual & 15)) return (int)cudaErrorInvalidValue;
      sp.residual = (const __nv_bfloat16*)epi->residual;
      sp.residual_ld = epi->residual_ld;
    }
    if (epi->rope_cos != nullptr) {
      if (!ROPE || SCATTER == 1 || epi->rope_sin == nullptr || epi->rope_period_cols <= 0 || (epi->rope_period_cols % 128) ||
          (epi->rope_rot_cols % 128) || epi->rope_rot_cols < 0 || epi->rope_rot_cols > epi->rope_period_cols || (N % 128) ||
          ((uintptr_t)epi->rope_cos & 15) || ((uintptr_t)epi->rope_sin & 15))
        return (int)cudaErrorInvalidValue;
      rp.cos = epi->rope_cos;
      rp.sin = epi->rope_sin;
      rp.period_cols = epi->rope_period_cols;
      rp.rot_cols = epi->rope_rot_cols;
    }
  }
  if ((r = make_tmap_2d_bf16(&tC, C, (uint64_t)N, (uint64_t)(SCATTER == 1 ? sd->chunk_rows : M), (uint64_t)ldc * 2, EPI_COLS, BM))) return 720000 + r;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int n_gemm = g_sms;
  if (tiles < n_gemm) n_gemm = tiles;
  if (GATHER && (gd->n_cta != n_gemm || (pd != nullptr && pd->n_cta != n_gemm))) return (int)cudaErrorInvalidConfiguration;   // the host's running totals assume this grid
  if (SCATTER) { sp.reduce_target = (uint32_t)n_gemm * sd->uses; sp.arrived_target = (uint32_t)n_gemm * sd->uses; }
  gemm_comm_kernel<LAYOUT, GATHER, SCATTER, ROPE><<<n_gemm, (GATHER && has_push) ? NUM_THREADS + COMM_THREADS : NUM_THREADS, SMEM_TOTAL, st>>>(tA, tB, tC, gp, pp, sp, M, N, K, ldc,
                                                                                           n_gemm, mn3d, rp, err);
  return (int)cudaGetLastError();
}

}  // namespace gc
}  // namespace ody

// gather / scatter may be null when that half is not used.  gather->which selects the gathered operand; push is
// the shard this launch's comm warps deliver (null: none - the operand was pushed by an earlier launch).
extern "C" int ody_gemm_comm_ex(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                                int64_t ldc, int layout, const OdyGatherDesc* gd, const OdyGatherDesc* pd,
                                const OdyScatterDesc* sd, const OdyEpilogue* epi, int* err, cudaStream_t st) {
  using namespace ody::gc;
  if (M <= 0 || N <= 0 || K <= 0 || (lda % 8) || (ldb % 8) || (N % 8)) return (int)cudaErrorInvalidValue;
  const int g = gd ? gd->which : 0;
  const int s = sd ? (sd->mode == 2 ? 2 : 1) : 0;
  const bool rope = epi != nullptr && epi->rope_cos != nullptr;
#define ODY_CASE(L, G, S) \
  if (layout == L && g == G && s == S && !rope) return launch<L, G, S, false>(A, B, C, M, N, K, lda, ldb, ldc, gd, pd, sd, epi, err, st);
#define ODY_CASE_ROPE(L, G, S) \
  if (layout == L && g == G && s == S && rope) return launch<L, G, S, true>(A, B, C, M, N, K, lda, ldb, ldc, gd, pd, sd, epi, err, st);
  ODY_CASE(0, 1, 0) ODY_CASE(0, 2, 0) ODY_CASE(1, 1, 0) ODY_CASE(1, 2, 0) ODY_CASE(2, 2, 0) ODY_CASE(2, 1, 0)
  ODY_CASE(0, 0, 1) ODY_CASE(1, 0, 1) ODY_CASE(2, 0, 1)
  ODY_CASE(0, 2, 2) ODY_CASE(1, 2, 2)
  // forward projections only: sequence gather -> q|k|v, weight gather -> q|k|v, weight gather -> q|k|v -> all-to-all
  ODY_CASE_ROPE(0, 1, 0) ODY_CASE_ROPE(0, 2, 0) ODY_CASE_ROPE(0, 2, 2)
#undef ODY_CASE_ROPE
#undef ODY_CASE
  return (int)cudaErrorInvalidValue;
}

extern "C" int ody_gemm_comm(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                             int64_t ldc, int layout, const OdyGatherDesc* gd, const OdyGatherDesc* pd,
                             const OdyScatterDesc* sd, int* err, cudaStream_t st) {
  return ody_gemm_comm_ex(A, B, C, M, N, K, lda, ldb, ldc, layout, gd, pd, sd, nullptr, err, st);
}

// Deliver a shard into every rank's gathered buffer without a GEMM (n_cta CTAs of 128 threads).
extern "C" int ody_push_shard(const OdyGatherDesc* pd, int* err, cudaStream_t st) {
  using namespace ody::gc;
  GatherParams pp;
  memset(&pp, 0, sizeof(pp));
  int r = fill_gather(pp, pd);
  if (r) return r;
  if (pd->shard == nullptr || (pd->shard_ld % 8) || ((uintptr_t)pd->shard & 15) || pd->n_cta <= 0) return (int)cudaErrorInvalidValue;
  push_shard_kernel<<<pd->n_cta, COMM_THREADS, 0, st>>>(pp, err);
  return (int)cudaGetLastError();
}

namespace ody {
namespace gc {
__global__ void wait_shard_kernel(const uint32_t* counter, uint32_t target, int* err, unsigned long long* acc) {
  __shared__ int abort_flag;
  abort_flag = 0;
  const unsigned long long t0 = acc ? global_ns() : 0;
  wait_word<true>(counter, target, &abort_flag, err, ODY_ERR_TIMEOUT_PEER);
  if (acc) atomicAdd(acc + 2, global_ns() - t0);     // the stream does nothing else meanwhile: all of it is exposed
}
struct PtrList { uint32_t* p[MAX_RANKS]; };
__global__ void wait_flags_kernel(const uint32_t* base, uint32_t mask, uint32_t target, int* err, unsigned long long* acc) {
  __shared__ int abort_flag;
  if (threadIdx.x == 0) abort_flag = 0;
  __syncthreads();
  const unsigned long long t0 = acc ? global_ns() : 0;
  if ((mask >> threadIdx.x) & 1u) wait_word<true>(base + threadIdx.x, target, &abort_flag, err, ODY_ERR_TIMEOUT_PEER);
  __syncthreads();
  if (acc && threadIdx.x == 0) atomicAdd(acc + 2, global_ns() - t0);
}
__global__ void signal_flags_kernel(const __grid_constant__ PtrList l, uint32_t mask, int index, uint32_t value) {
  __threadfence_system();
  if ((mask >> threadIdx.x) & 1u) st_release_sys(l.p[threadIdx.x] + index, value);
}
__global__ void signal_free_kernel(const __grid_constant__ GatherParams g) {
  __threadfence_system();
  if ((int)threadIdx.x < g.n_ranks) st_release_sys(g.free_peer[threadIdx.x] + g.rank, g.epoch);
}
}  // namespace gc
}  // namespace ody

extern "C" int ody_wait_shard(const OdyGatherDesc* d, int src, int* err, cudaStream_t st) {
  using namespace ody::gc;
  if (d == nullptr || src < 0 || src >= d->n_ranks) return (int)cudaErrorInvalidValue;
  wait_shard_kernel<<<1, 1, 0, st>>>(d->counters_peer[d->rank] + src, d->push_total, err, wait_acc_here());
  return (int)cudaGetLastError();
}

extern "C" int ody_wait_flags(const uint32_t* base, uint32_t mask, uint32_t target, int* err, cudaStream_t st) {
  if (base == nullptr) return (int)cudaErrorInvalidValue;
  if (mask == 0) return 0;
  ody::gc::wait_flags_kernel<<<1, 32, 0, st>>>(base, mask, target, err, ody::gc::wait_acc_here());
  return (int)cudaGetLastError();
}

extern "C" int ody_signal_flags(uint32_t* const* ptrs, int n, uint32_t mask, int index, uint32_t value, cudaStream_t st) {
  using namespace ody::gc;
  if (n < 1 || n > MAX_RANKS || (mask >> n) != 0 || index < 0) return (int)cudaErrorInvalidValue;
  if (mask == 0) return 0;
  PtrList l;
  for (int p = 0; p < MAX_RANKS; ++p) l.p[p] = p < n ? ptrs[p] : nullptr;
  signal_flags_kernel<<<1, 32, 0, st>>>(l, mask, index, value);
  return (int)cudaGetLastError();
}

extern "C" int ody_signal_free(const OdyGatherDesc* d, cudaStream_t st) {
  using namespace ody::gc;
  GatherParams g;
  memset(&g, 0, sizeof(g));
  int r = fill_gather(g, d);
  if (r) return r;
  signal_free_kernel<<<1, 32, 0, st>>>(g);
  return (int)cudaGetLastError();
}

// acc: device uint64[4] on the current device that the fused kernels add their waiting times to (ns), or NULL to stop:
// [0] gather GEMMs, summed over CTAs: TMA producers waiting for remote rows; [1] reduce-scatter GEMMs, one thread per
// CTA: owners waiting for the sources' tiles; [2] the stand-alone wait kernels (the stream is idle for all of it).
extern "C" int ody_set_wait_accumulator(unsigned long long* acc) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
  ody::gc::g_wait_acc[dev] = acc;
  return 0;
}

extern "C" int ody_set_push_order(int unit_major) {
  const int v = unit_major ? 1 : 0;
  int r = (int)cudaMemcpyToSymbol(ody::gc::g_push_unit_major, &v, sizeof(v));
  if (r) return r;
  return ody_flash_set_push_order(v);
}

extern "C" int ody_set_peer_wait_limit(long long cycles) {
  if (cycles <= 0) return (int)cudaErrorInvalidValue;
  int r = (int)cudaMemcpyToSymbol(ody::gc::g_peer_spin_limit, &cycles, sizeof(cycles));
  if (r) return r;
  return ody_flash_set_peer_wait_limit(cycles);
}
