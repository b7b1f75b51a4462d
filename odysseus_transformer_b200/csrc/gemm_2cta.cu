// bf16 GEMM for sm_100a on CTA PAIRS: tcgen05.mma.cta_group::2 inside clusters of two.
//
// Same contract as gemm.cu (the GEMM core behind every linear layer; the reference reaches cuBLAS through
// torch.matmul / F.linear: reference utils/linear_tpsp.py:173,217,291,588; utils/linear_zero3.py:44,68,74):
//
//   layout 0 (NT): C[M,N] = A[M,K] * B[N,K]^T      layout 1 (NN): C = A[M,K] * B[K,N]      layout 2 (TN): C = A[K,M]^T * B[K,N]
//
// Two CTAs on neighbouring SMs share one 256 x 256 output tile.  Each holds 128 rows of A and HALF of the B tile
// (128 of its 256 columns) per 64-deep k-block in its own shared memory - 32 KB per stage instead of the 48 KB a
// single CTA needs for 128 x 256 - and ONE thread of the even CTA issues 256 x 256 x 16 instructions that read both
// halves and accumulate 128 x 256 fp32 in the tensor memory of each SM.  Per output element the tensor core reads
// a third less shared memory and L2 than the one-CTA kernel, which is what that kernel is bound by.
//
// Protocol.  Every TMA load is a plain (non-multicast) load of this GPU's memory into the issuing CTA's own shared
// memory; with .cta_group::2 it signals the EVEN CTA's `full` barrier, whose transaction count covers the bytes of
// both CTAs.  The issuing thread frees a stage with a tcgen05.commit that arrives on the `empty` barrier of both
// CTAs (commit multicast, not a load), and publishes a finished accumulator the same way.  Each CTA's four epilogue
// warps drain their own 128 rows, store them with TMA, and tell the even CTA (remote mbarrier arrive) that the
// accumulator buffer is free.  Two 256-column accumulators alternate, so the epilogue overlaps the next main loop.
// Every wait is bounded; the cluster barriers at start and end are the only unbounded synchronisation, and every
// thread reaches them on every path.
#include "ody_kernels.h"
#include "sm100.cuh"

// defined in gemm.cu: validates an epilogue description and resolves it into kernel arguments
extern "C" int ody_gemm_resolve_epilogue(const OdyEpilogue* epi, const void* C, int M, int N, int64_t ldc, int* accumulate,
                                         const void** c_in, int64_t* ld_in, ody::RopeEpi* rp);

namespace ody {
namespace g2 {

constexpr int BM = 128;                          // rows per CTA (256 per pair)
constexpr int BN = 256;                          // columns of the pair's tile
constexpr int BNH = BN / 2;                      // B columns held by each CTA
constexpr int BK = 64, STAGES = 5, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;             // 16 KB
constexpr int B_BYTES = BNH * BK * 2;            // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // 32 KB per CTA
constexpr int EPI_COLS = 64;
constexpr int EPI_BYTES = BM * EPI_COLS * 2;     // 16 KB
constexpr int SMEM_TILES = STAGES * STAGE_BYTES + 2 * EPI_BYTES;
constexpr int SMEM_TOTAL = SMEM_TILES + 256 + 1024;
constexpr int NUM_THREADS = 192;                 // TMA warp, MMA warp, 4 epilogue warps
constexpr int GROUP_M = 8;                       // raster: 8 pair-tiles (2048 rows) share their B columns in L2

struct Bars {
  uint64_t full[STAGES];        // used in the even CTA only
  uint64_t empty[STAGES];       // one per CTA, both raised by the issuer's commit
  uint64_t tmem_full[2];        // one per CTA, both raised by the issuer's commit
  uint64_t tmem_empty[2];       // used in the even CTA only: 128 local + 128 remote arrivals
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `p` (a location in this CTA's shared memory) as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA loads of a CTA pair: destination in the issuing CTA, completion counted on `bar_cluster_addr` (the even CTA's
// barrier).  No multicast: each CTA fetches only what it alone needs, from this GPU's own memory.
__device__ __forceinline__ void tma2_load_2d(void* smem_dst, const CUtensorMap* tmap, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(x), "r"(y), "r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* smem_dst, const CUtensorMap* tmap, int x, int y, int z, uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tmem2_alloc(uint32_t* smem_result, uint32_t ncols) {   // one whole warp in EACH CTA
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem2_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem2_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[128 rows in each CTA] * B[half the columns in each CTA]; one thread of the even CTA issues
__device__ __forceinline__ void umma2_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// arrives, once all MMAs issued so far have completed, on the barrier at this shared-memory offset in BOTH CTAs
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}

// same, arriving on this CTA's barrier only
__device__ __forceinline__ void umma2_commit_local(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsize = min(GROUP_M, tiles_m - first_m);
  const int local = tile - g * per_group;
  tm = first_m + local % gsize;
  tn = local / gsize;
}

__device__ __forceinline__ bool epi_all_ok(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 2, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(r)
      : "r"((uint32_t)ok)
      : "memory");
  return r != 0;
}

// ROPE: the epilogue rotates the q / k heads of a packed projection (RopeEpi, sm100.cuh); a separate instance, so that
// the plain one keeps its register allocation
template <int LAYOUT, bool ROPE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, const __nv_bfloat16* __restrict__ c_in, int M, int N, int K,
                  int64_t ldc, int accumulate, int mn3d, const RopeEpi rp, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Bars* bars = (Bars*)(smem + SMEM_TILES);
  uint8_t* epi = smem + STAGES * STAGE_BYTES;
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();            // 0: issues the MMAs and owns the full / tmem_empty barriers
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (K + BK - 1) / BK;
  constexpr bool A_MN = (LAYOUT == 2), B_MN = (LAYOUT != 0);
  constexpr uint32_t IDESC = make_idesc_bf16(2 * BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->tmem_full[b], 1);
      mbar_init(&bars->tmem_empty[b], 256);
    }
    mbar_init(&bars->drain, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmC);
  }
  if (warp == 1) {
    tmem2_alloc(&bars->tmem_base, 512);
    tmem2_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers exist before anything may signal them from the other side
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (each CTA loads its own halves)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * 2 * BM + (int)rank * BM;        // this CTA's rows of A
        const int n0 = tn * BN + (int)rank * BNH;           // this CTA's columns of B
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sA = smem + stage * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          if (rank == 0) mbar_expect_tx(&bars->full[stage], 2 * STAGE_BYTES);     // the bytes of both CTAs
          const uint32_t full0 = map_to_cta(&bars->full[stage], 0);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma2_load_2d(sA, &tmA, k0, m0, full0);
          } else if (mn3d & 1) {
            tma2_load_3d(sA, &tmA, 0, k0, m0 / 64, full0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma2_load_2d(sA + j * 8192, &tmA, m0 + 64 * j, k0, full0);
          }
          if (!B_MN) {
            tma2_load_2d(sB, &tmB, k0, n0, full0);
          } else if (mn3d & 2) {
            tma2_load_3d(sB, &tmB, 0, k0, n0 / 64, full0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma2_load_2d(sB + j * 8192, &tmB, n0 + 64 * j, k0, full0);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if ((!ok || *abort_flag) && rank == 0) {
        // give copies still in flight a bounded chance to land before the CTA retires
        int n = issued < STAGES ? issued : STAGES;
        for (int i = 0; i < n; ++i) {
          if (--stage < 0) { stage = STAGES - 1; phase ^= 1; }
          const long long t0 = clock64();
          while (!mbar_try_wait(&bars->full[stage], phase) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    if (rank == 0) {
      // every lane runs the control flow, so the compiler keeps descriptors and loop state in uniform registers and an MMA
      // costs a few instructions; one elected lane issues the tcgen05 instructions (benchmarks/mma_issue_rate.cu)
      const bool leader = elect_one();
      int stage = 0;
      uint32_t phase = 0;
      int local_tile = 0;
      bool ok = true;
      const uint32_t s0 = smem_u32(smem);
      const uint64_t adesc0 = A_MN ? make_smem_desc(s0, 8192, 1024) : make_smem_desc(s0, 16, 1024);
      const uint64_t bdesc0 = B_MN ? make_smem_desc(s0 + A_BYTES, 8192, 1024) : make_smem_desc(s0 + A_BYTES, 16, 1024);
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++local_tile) {
        const int buf = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[buf], acc_phase ^ 1, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, abort_flag, err, ODY_ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint64_t a0 = desc_advance(adesc0, stage * STAGE_BYTES), b0 = desc_advance(bdesc0, stage * STAGE_BYTES);
          if (leader) umma2_ss(d_tmem, a0, b0, IDESC, kb > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < BK / UMMA_K; ++kk)
            if (leader) umma2_ss(d_tmem, desc_advance(a0, kk * (A_MN ? 2048 : 32)), desc_advance(b0, kk * (B_MN ? 2048 : 32)), IDESC, 1u);
          if (leader) umma2_commit_both(&bars->empty[stage]);      // frees the stage in both CTAs once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok && leader) umma2_commit_both(&bars->tmem_full[buf]);   // accumulators of both CTAs complete
      }
      if (!ok || *abort_flag) {
        if (leader) umma2_commit_local(&bars->drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(&bars->drain, 0) && clock64() - t0 < ODY_SPIN_LIMIT_CYCLES / 8) {}
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of each CTA: its own 128 rows)
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int r = q * 32 + lane;                 // row inside this CTA's half of the tile
    const bool store_thread = (warp == 2 && lane == 0);
    int local_tile = 0;
    for (int tile = pair; tile < num_tiles; tile += n_pairs, ++local_tile) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      const int m0 = tm * 2 * BM + (int)rank * BM, n0 = tn * BN;
      const int buf = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      bool ok = mbar_wait(&bars->tmem_full[buf], acc_phase, abort_flag, err, ODY_ERR_TIMEOUT_TMEM_FULL);
      if (!epi_all_ok(ok)) break;
      tc_fence_after();
      const uint32_t empty0 = map_to_cta(&bars->tmem_empty[buf], 0);
#pragma unroll 1
      for (int c = 0; c < BN / EPI_COLS; ++c) {
        uint8_t* sbuf = epi + (c & 1) * EPI_BYTES;
        if (store_thread) tma_store_wait_read<1>();
        named_barrier(1, 128);
        const uint32_t taddr = tmem_base + buf * BN + c * EPI_COLS + ((uint32_t)(q * 32) << 16);
        uint32_t v[64];
        tmem_ld_32x32(taddr, v);
        tmem_ld_32x32(taddr + 32, v + 32);
        tmem_ld_wait();
        const int row = m0 + r, col0 = n0 + c * EPI_COLS;
        if (ROPE && rope_epi_wants(rp, col0)) {
          // the other half of this head, still in the accumulator (read before the buffer is handed back below)
          uint32_t w[64];
          const uint32_t paddr = (c & 1) ? taddr - EPI_COLS : taddr + EPI_COLS;
          tmem_ld_32x32(paddr, w);
          tmem_ld_32x32(paddr + 32, w + 32);
          tmem_ld_wait();
          if (row < M) rope_epi_apply(rp, row, c & 1, v, w);
        }
        if (c == BN / EPI_COLS - 1) {
          tc_fence_before();
          mbar_arrive_cluster(empty0);            // this thread's rows of the accumulator are in registers
        }
        if (accumulate && row < M) {
          const __nv_bfloat16* cp = c_in + (int64_t)row * ldc + col0;
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
        if (store_thread && col0 < N && m0 < M) {
          tma_store_2d(&tmC, sbuf, col0, m0);
          tma_store_commit();
        }
      }
    }
    if (store_thread) tma_store_wait<0>();
  }

  // neither CTA may retire while the other can still read its shared memory (operands of a pair MMA) or signal its barriers
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem2_dealloc(tmem_base, 512);
  }
}

static int g_max_pairs = 0;

template <int LAYOUT, bool ROPE>
static int launch(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                  int accumulate, const void* c_src, int64_t ld_in, const RopeEpi& rp, int* err, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm2_bf16_kernel<LAYOUT, ROPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = SMEM_TOTAL;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (g_max_pairs == 0) {
    int dev = 0, sms = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cfg.gridDim = dim3(sms - (sms & 1));
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm2_bf16_kernel<LAYOUT, ROPE>, &cfg);
    if (e != cudaSuccess || n <= 0) { cudaGetLastError(); n = sms / 2; }     // fall back to the nominal count
    g_max_pairs = n < sms / 2 ? n : sms / 2;
  }
  CUtensorMap tA, tB, tC;
  int r;
  int mn3d = 0;   // bit 0: A tile is one blocked 3-D TMA load, bit 1: B tile is
  if (LAYOUT == 2 && (M % 64) == 0) { r = make_tmap_mn_blocked_bf16(&tA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, BK, BM / 64); mn3d |= 1; }
  else if (LAYOUT == 2) r = make_tmap_2d_bf16(&tA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, 64);
  else r = make_tmap_2d_bf16(&tA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, 64, BM);
  if (r) return 700000 + r;
  if (LAYOUT == 0) r = make_tmap_2d_bf16(&tB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, 64, BNH);
  else if ((N % 64) == 0) { r = make_tmap_mn_blocked_bf16(&tB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, BK, BNH / 64); mn3d |= 2; }
  else r = make_tmap_2d_bf16(&tB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, 64);
  if (r) return 710000 + r;
  r = make_tmap_2d_bf16(&tC, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, EPI_COLS, BM);
  if (r) return 720000 + r;
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  const int pairs = tiles < g_max_pairs ? tiles : g_max_pairs;
  cfg.gridDim = dim3(2 * pairs);
  const __nv_bfloat16* c_in = (const __nv_bfloat16*)c_src;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm2_bf16_kernel<LAYOUT, ROPE>, tA, tB, tC, c_in, M, N, K, ld_in, accumulate, mn3d, rp, err);
  return (int)e;
}

}  // namespace g2
}  // namespace ody

// Same arguments as ody_gemm_bf16_ex; the pair kernel.  ody_gemm_bf16_ex chooses between the two (gemm.cu).
extern "C" int ody_gemm_bf16_2cta_ex(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                                     int64_t ldc, int layout, int accumulate, const OdyEpilogue* epi, int* err,
                                     cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return (int)cudaErrorInvalidValue;
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)C & 15))
    return (int)cudaErrorInvalidValue;
  const void* c_in;
  int64_t ld_in;
  ody::RopeEpi rp;
  if (int r = ody_gemm_resolve_epilogue(epi, C, M, N, ldc, &accumulate, &c_in, &ld_in, &rp)) return r;
  if (rp.cos != nullptr)   // a forward projection: layout 0 only
    return layout == 0 ? ody::g2::launch<0, true>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, c_in, ld_in, rp, err, st)
                       : (int)cudaErrorInvalidValue;
  switch (layout) {
    case 0: return ody::g2::launch<0, false>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, c_in, ld_in, rp, err, st);
    case 1: return ody::g2::launch<1, false>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, c_in, ld_in, rp, err, st);
    case 2: return ody::g2::launch<2, false>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, c_in, ld_in, rp, err, st);
  }
  return (int)cudaErrorInvalidValue;
}

extern "C" int ody_gemm_bf16_2cta(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                                  int64_t ldc, int layout, int accumulate, int* err, cudaStream_t st) {
  return ody_gemm_bf16_2cta_ex(A, B, C, M, N, K, lda, ldb, ldc, layout, accumulate, nullptr, err, st);
}
