// Peer-memory building blocks shared by the fused kernels: the description of a gathered buffer, bounded
// polls of epoch words, system-scope release/acquire helpers, and the "comm warps" that push this rank's
// shard into every rank's gathered buffer with plain 16-byte stores over NVLink.
//
// Waits on peers may legitimately last as long as another rank is behind (first-step set-up, host jitter),
// so their bound is a run-time setting, one copy per translation unit (default about 10 s of SM clocks)
// instead of the 1 s used by waits on this GPU's own pipeline.
#pragma once
#include <string.h>

#include "ody_kernels.h"

namespace ody { namespace gc {
static __device__ long long g_peer_spin_limit = 20000000000ll;
// 0: serve the destinations one after the other (default); 1: every unit to all destinations at once.  A run-time
// switch so that the two schedules can be timed against each other (benchmarks/comm_bench.py --push-order).
static __device__ int g_push_unit_major = 0;
} }

#include "sm100.cuh"

namespace ody {
namespace gc {

constexpr int MAX_RANKS = 8;
constexpr int COMM_THREADS = 128;         // four comm warps: three move data, one fences and signals

struct GatherParams {
  __nv_bfloat16* gathered_peer[MAX_RANKS];   // rank p's gathered buffer [n_ranks * chunk_rows, cols], dense
  const __nv_bfloat16* shard;                // this rank's shard [chunk_rows, cols], row pitch shard_ld
  int64_t shard_ld;
  uint32_t* flags_peer[MAX_RANKS];     // rank p's arrival counters, one per unit_rows-row block of its gathered buffer
  uint32_t* counters_peer[MAX_RANKS];  // rank p's per-source "whole shard delivered" counters
  uint32_t* free_peer[MAX_RANKS];      // free_peer[p][rank] <- epoch : "rank `rank` has finished reading its gathered buffer"
  uint32_t* flags_local;
  uint32_t* counters_local;
  uint32_t* free_local;         // [n_ranks] epochs written by the consumers of my pushes
  uint32_t* gemm_done;          // local counter of CTAs that finished (the last one frees the buffer)
  int n_ranks, rank, chunk_rows, cols;
  int unit_rows;                // 128, or 64 when chunk_rows is only a multiple of 64
  int unit_cols;                // 256, or 64 when cols is only a multiple of 64
  int dest_first, dest_count;   // destinations are ranks rank + dest_first, ..., rank + dest_first + dest_count - 1 (mod n_ranks)
  uint32_t epoch;               // this use of the buffer
  uint32_t prev_epoch;          // previous use of the same buffer (its readers must be done)
  uint32_t flag_target;         // cumulative: (cols / unit_cols) * uses
  uint32_t counter_target;      // cumulative: CTAs per launch summed over uses
  uint32_t gemm_done_target;    // same number: every CTA reports once per launch
  unsigned long long* stats;    // optional [n_cta][4] ns: comm begin, comm end, time the producer spent waiting for rows, CTA end
  unsigned long long* wait_acc; // optional running totals (ns): [0] += the time this launch's producers waited for remote rows
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded poll of a monotonically increasing word: true once *p - target is non-negative (wrap-safe).
template <bool SYS>
__device__ __forceinline__ bool wait_word(const uint32_t* p, uint32_t target, volatile int* abort_flag, int* err, int code) {
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    const uint32_t v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if ((int32_t)(v - target) >= 0) return true;
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > g_peer_spin_limit) {
        if (err != nullptr) atomicCAS(err, 0, code);
        *abort_flag = 1;
        return false;
      }
    }
    __nanosleep(64);
  }
}

// ------------------------------------------------------------------------------------------- comm warps
// The comm warps of CTA `cta` (of n_cta) push units cta, cta + n_cta, ... of this rank's shard.
// unit = unit_rows x unit_cols elements.  Three data warps move 16-byte vectors, 8 loads in flight per
// thread.  The fourth warp is the signaler: once the data warps have issued a unit (named barrier) it
// fences at system scope - which waits for those stores to be acknowledged - and bumps that row block's
// arrival counter at the destination(s), while the data warps are already moving the next unit.
constexpr int DATA_THREADS = COMM_THREADS - 32;
static __device__ void comm_warps_main(const GatherParams& g, int cta, int n_cta, int first_thread, volatile int* abort_flag, int* err) {
  const int ct = threadIdx.x - first_thread;
  const bool signaler = ct >= DATA_THREADS;
  const int UR = g.unit_rows, UC = g.unit_cols;
  const int nb = g.chunk_rows / UR;
  const int boxes = g.cols / UC;
  const int total_units = nb * boxes;
  const int vpr = UC / 8;                       // vectors per unit row
  const int nvec = UR * vpr;
  const int64_t my_row0 = (int64_t)g.rank * g.chunk_rows;
  if (g.stats != nullptr && ct == 0) g.stats[cta * 4 + 0] = global_ns();
  bool ok = true;
  // every destination other than this rank must have finished reading this slot's last contents
  if (ct < g.n_ranks && ct != g.rank && (ct - g.rank + g.n_ranks - g.dest_first) % g.n_ranks < g.dest_count)
    ok = wait_word<true>(g.free_local + ct, g.prev_epoch, abort_flag, err, ODY_ERR_TIMEOUT_PEER);
  {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 3, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(r) : "r"((uint32_t)ok) : "memory");
    if (!r) return;
  }
  // Schedule.  Destination-major (default): the destinations are served one after the other, every unit of this CTA
  // to the first before any to the second; when the shard goes to every rank the order is own, rank - 1, rank - 2,
  // ...  A consumer walks the gathered rows upwards from its own shard, so the first data it needs from another
  // rank are those of rank + 1, and this way it receives them first, at the full rate of that source, instead of an
  // equal trickle from all sources that completes everywhere at the same late moment.  Unit-major: every unit is
  // read once and stored to all destinations.
  const bool everyone = g.dest_first == 0 && g.dest_count == g.n_ranks;
  const bool unit_major = g_push_unit_major != 0;
  auto dest = [&](int s) { return everyone ? (g.rank - s + g.n_ranks) % g.n_ranks : (g.rank + g.dest_first + s) % g.n_ranks; };
  const int rounds = unit_major ? 1 : g.dest_count;          // destination groups served one after the other
  const int per_round = unit_major ? g.dest_count : 1;
  for (int round = 0; round < rounds; ++round) {
    const int s0 = round * per_round;
    for (int u = cta; u < total_units; u += n_cta) {
      const int blk = u / boxes, cb = u % boxes;
      if (!signaler) {
        for (int v0 = ct; v0 < nvec; v0 += DATA_THREADS * 8) {
          uint4 val[8];
          int64_t dst_off[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int v = v0 + i * DATA_THREADS;
            const int row = v / vpr, cv = v % vpr;
            const int64_t rr = (int64_t)blk * UR + row;
            dst_off[i] = (my_row0 + rr) * g.cols + cb * UC + cv * 8;
            if (v < nvec) val[i] = *reinterpret_cast<const uint4*>(g.shard + rr * g.shard_ld + cb * UC + cv * 8);
          }
          for (int s = s0; s < s0 + per_round; ++s) {
            __nv_bfloat16* base = g.gathered_peer[dest(s)];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (v0 + i * DATA_THREADS < nvec) *reinterpret_cast<uint4*>(base + dst_off[i]) = val[i];
          }
        }
      }
      named_barrier(3, COMM_THREADS);            // unit u has been issued by every data thread
      if (ct == DATA_THREADS) {
        __threadfence_system();
        for (int s = s0; s < s0 + per_round; ++s) red_release_sys_add(g.flags_peer[dest(s)] + g.rank * nb + blk, 1);
      }
    }
    if (ct == DATA_THREADS) {
      __threadfence_system();
      for (int s = s0; s < s0 + per_round; ++s) red_release_sys_add(g.counters_peer[dest(s)] + g.rank, 1);
    }
  }
  if (ct == DATA_THREADS && g.stats != nullptr) g.stats[cta * 4 + 1] = global_ns();
}



// Host side: translate a description into kernel parameters.
static inline int fill_gather(GatherParams& g, const OdyGatherDesc* d) {
  if (d == nullptr || d->n_ranks < 2 || d->n_ranks > MAX_RANKS || (d->cols % 64) || (d->chunk_rows % 64)) return (int)cudaErrorInvalidValue;
  for (int p = 0; p < d->n_ranks; ++p) {
    g.gathered_peer[p] = (__nv_bfloat16*)d->gathered_peer[p];
    g.flags_peer[p] = d->flags_peer[p];
    g.counters_peer[p] = d->counters_peer[p];
    g.free_peer[p] = d->free_peer[p];
  }
  g.shard = (const __nv_bfloat16*)d->shard;
  g.shard_ld = d->shard_ld;
  g.flags_local = d->flags_peer[d->rank];
  g.counters_local = d->counters_peer[d->rank];
  g.free_local = d->free_peer[d->rank];
  g.gemm_done = d->gemm_done;
  g.n_ranks = d->n_ranks; g.rank = d->rank; g.chunk_rows = d->chunk_rows; g.cols = d->cols;
  g.unit_rows = (d->chunk_rows % 128) ? 64 : 128;   // a unit never straddles two shards
  g.unit_cols = (d->cols % 256) ? 64 : 256;
  g.dest_first = d->dest_count > 0 ? d->dest_first : 0;
  g.dest_count = d->dest_count > 0 ? d->dest_count : d->n_ranks;
  if (g.dest_first < 0 || g.dest_first + g.dest_count > d->n_ranks) return (int)cudaErrorInvalidValue;
  g.epoch = d->epoch; g.prev_epoch = d->prev_epoch;
  g.flag_target = (uint32_t)(d->cols / g.unit_cols) * d->uses;
  g.counter_target = d->push_total;
  g.gemm_done_target = d->consume_total;
  g.stats = (unsigned long long*)d->stats;
  return 0;
}


}  // namespace gc
}  // namespace ody
