// Micro-benchmark: SM cycles per tcgen05.mma instruction (bf16, M = 128, cta_group::1) as seen by the issuing thread,
// for the operand forms the attention kernels use, alone and next to arithmetic warps on the same schedulers.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr \
//        -I odysseus_transformer_b200/csrc benchmarks/mma_issue_rate.cu -o mma_issue_rate -lcuda && ./mma_issue_rate
//
// One CTA per SM; thread 0 issues 400 chains of eight instructions (the issue of an instruction blocks while the pipe's
// queue is full, so cycles / instruction of the loop is the execution rate) and waits for their completion through a
// bounded mbarrier wait.  Variants: both operands from shared memory (SS) or A from TMEM (TS), B K-major or MN-major,
// one to three accumulators, N = 128 or 256, chains whose A columns the next chain overwrites, two issuing warps, and
// eight extra warps that stream tcgen05.ld, or run dense FMA + MUFU code (sixteen independent chains per thread), with
// and without a pause every ~20 instructions; and the issuing loop run by the whole warp with one elected lane issuing
// (warp-uniform control flow) instead of under `if (lane == 0)`.  What it shows: the pipe takes a 128 x 128 x 16 instruction every 64 cycles
// in every operand form; a lone issuing warp next to dense arithmetic warps gets one out only every ~99 cycles when the
// loop runs under `if (lane == 0)`, and every 64 when it runs warp-uniformly.
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include "ody_kernels.h"
#include "sm100.cuh"

using namespace ody;

struct PBars { uint64_t done; uint64_t done2; uint32_t tmem_base; int abort_flag; };

// KIND 0: SS, B K-major; 1: SS, B MN-major; 2: TS, B K-major; 3: TS, B MN-major.  LD: 8 extra warps stream tcgen05.ld meanwhile.
template <int KIND, int N, int NACC, bool LD, bool MATH = false, int YIELD = 0, bool UNI = false>
__global__ void __launch_bounds__(384, 1) probe(int groups, long long* out, int* err) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = 128 * 256, B_BYTES = N * 256, NB = 3;
  uint8_t* sA = smem;
  uint8_t* sB = smem + A_BYTES;
  PBars* bars = (PBars*)(smem + A_BYTES + NB * B_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (A_BYTES + NB * B_BYTES) / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0x3c003c00u + (i & 0xff);
  if (threadIdx.x == 0) { mbar_init(&bars->done, 1); mbar_init(&bars->done2, 1); bars->abort_flag = 0; mbar_fence_init(); }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  volatile int* abort_flag = &bars->abort_flag;
  if (UNI && warp == 0) {
    constexpr uint32_t IDESC = make_idesc_bf16(128, N, 0, 0);
    const uint32_t acol = NACC * N;
    const long long t0 = clock64();
    for (int g = 0; g < groups; ++g) {
      const uint32_t d = tmem + (g % NACC) * N;
      const uint64_t bk = make_smem_desc(smem_u32(sB) + (g % NB) * B_BYTES, 16, 1024);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t bd = desc_advance(bk, (kk >> 2) * (B_BYTES / 2) + (kk & 3) * 32);
        if (elect_one()) umma_ts(d, tmem + acol + kk * 8, bd, IDESC, 1u);
      }
    }
    const long long t1 = clock64();
    if (elect_one()) umma_commit(&bars->done);
    __syncwarp();
    mbar_wait(&bars->done, 0, abort_flag, err, 1);
    const long long t2 = clock64();
    if (blockIdx.x == 0 && lane == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  } else if (!UNI && warp == 0 && lane == 0) {
    constexpr uint32_t IDESC = make_idesc_bf16(128, N, 0, (KIND & 1) ? 1 : 0);
    const uint64_t a0 = make_smem_desc(smem_u32(sA), 16, 1024);
    const uint32_t acol = NACC * N;             // A operand columns (TS)
    const long long t0 = clock64();
    for (int g = 0; g < groups; ++g) {
      const uint32_t d = tmem + (g % NACC) * N;
      const uint32_t boff = (g % NB) * B_BYTES;
      const uint64_t bk = make_smem_desc(smem_u32(sB) + boff, 16, 1024);
      const uint64_t bmn = make_smem_desc(smem_u32(sB) + boff, 128 * 128, 1024);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t bd = (KIND & 1) ? desc_advance(bmn, kk * 2048) : desc_advance(bk, (kk >> 2) * (B_BYTES / 2) + (kk & 3) * 32);
        if (KIND == 4 || KIND == 5) {
          // even groups: D = columns 256.., A read from columns 128.. (KIND 4) or from the operand columns (KIND 5);
          // odd groups: D = columns 128.. overwritten (first instruction does not accumulate), A from the operand columns
          if ((g & 1) == 0) umma_ts(tmem + 256, tmem + (KIND == 4 ? 128 : 448) + kk * 8, bd, IDESC, 1u);
          else umma_ts(tmem + 128, tmem + 384 + kk * 8, bd, IDESC, kk > 0 ? 1u : 0u);
        } else if (KIND == 7) {
          umma_ts(tmem, tmem + 384 + kk * 8, bd, IDESC, 1u);
        } else if (KIND == 6) {
          // one accumulator chain restarted every group (first instruction overwrites): no cross-operand hazard
          umma_ts(d, tmem + acol + kk * 8, bd, IDESC, kk > 0 ? 1u : 0u);
        } else if (KIND < 2) umma_ss(d, desc_advance(a0, (kk >> 2) * (A_BYTES / 2) + (kk & 3) * 32), bd, IDESC, 1u);
        else umma_ts(d, tmem + acol + kk * 8, bd, IDESC, 1u);
      }
    }
    const long long t1 = clock64();             // the issue loop blocks while the pipe is full: t1 - t0 ~ execution time
    umma_commit(&bars->done);
    mbar_wait(&bars->done, 0, abort_flag, err, 1);
    const long long t2 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  } else if (KIND == 7 && warp == 2 && lane == 0) {
    constexpr uint32_t IDESC = make_idesc_bf16(128, N, 0, 0);
    for (int g = 0; g < groups; ++g) {
      const uint64_t bk = make_smem_desc(smem_u32(sB) + (g % NB) * B_BYTES, 16, 1024);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_ts(tmem + 256, tmem + 448 + kk * 8, desc_advance(bk, (kk >> 2) * (B_BYTES / 2) + (kk & 3) * 32), IDESC, 1u);
    }
    umma_commit(&bars->done2);
    mbar_wait(&bars->done2, 0, abort_flag, err, 2);
    if (blockIdx.x == 0) out[2] = clock64();
  } else if (LD && warp >= 4) {
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t acc = 0;
    for (int i = 0; i < (MATH ? groups / 8 : groups * 2) && !*abort_flag; ++i) {
      uint32_t v[32];
      tmem_ld_32x32(tmem + ((i * 32) % (NACC * N)) + lane_off, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) acc ^= v[j];
      if (MATH) {
        // 16 independent chains: the warp can issue almost every cycle
        float x[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) x[u] = __uint_as_float(v[u] & 0x3fffffffu);
#pragma unroll 1
        for (int j = 0; j < 96; ++j) {
#pragma unroll
          for (int u = 0; u < 16; ++u) x[u] = fmaf(x[u], 1.0001f, 0.5f);
#pragma unroll
          for (int u = 0; u < 16; u += 4) x[u] = exp2_mufu(x[u] * 1e-3f);
          if (YIELD == 1) { x[0] += __uint_as_float(*(volatile uint32_t*)(smem + ((j * 4) & 1020))); }          // a dependent shared-memory load
          if (YIELD == 2) { __nanosleep(0); }
          if (YIELD == 3) { asm volatile("bar.warp.sync 0xffffffff;" ::: "memory"); }
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) acc ^= __float_as_uint(x[u]);
      } else {
        __nanosleep(200);
      }
    }
    if (acc == 0x12345u) out[3] = acc;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

template <int KIND, int N, int NACC, bool LD, bool MATH = false, int YIELD = 0, bool UNI = false>
void run(const char* name, int groups, long long* out, int* err) {
  constexpr int SMEM = 128 * 256 + 3 * N * 256 + 256 + 1024;
  cudaFuncSetAttribute(probe<KIND, N, NACC, LD, MATH, YIELD, UNI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  cudaMemset(out, 0, 32);
  for (int rep = 0; rep < 2; ++rep) probe<KIND, N, NACC, LD, MATH, YIELD, UNI><<<148, 384, SMEM>>>(groups, out, err);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[4]; int herr = 0;
  cudaMemcpy(h, out, 32, cudaMemcpyDeviceToHost);
  cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost);
  const double n = groups * 8.0;
  printf("%-44s issue %.1f cycles/instr, complete %.1f cycles/instr  (%s, status %d)\n", name, h[0] / n, h[1] / n,
         cudaGetErrorString(e), herr);
}

int main() {
  long long* out; int* err;
  cudaMalloc(&out, 32); cudaMalloc(&err, 4); cudaMemset(err, 0, 4);
  const int G = 400;
  run<0, 128, 3, false>("SS  N=128 B K-major, 3 accumulators", G, out, err);
  run<0, 128, 1, false>("SS  N=128 B K-major, 1 accumulator", G, out, err);
  run<1, 128, 3, false>("SS  N=128 B MN-major, 3 accumulators", G, out, err);
  run<2, 128, 3, false>("TS  N=128 B K-major, 3 accumulators", G, out, err);
  run<3, 128, 3, false>("TS  N=128 B MN-major, 3 accumulators", G, out, err);
  run<2, 128, 3, true>("TS  N=128 B K-major, 3 acc, tcgen05.ld traffic", G, out, err);
  run<0, 128, 3, true>("SS  N=128 B K-major, 3 acc, tcgen05.ld traffic", G, out, err);
  run<2, 128, 3, true, true>("TS  N=128, 8 warps of FMA + MUFU + tcgen05.ld", G, out, err);
  run<0, 128, 3, true, true>("SS  N=128, 8 warps of FMA + MUFU + tcgen05.ld", G, out, err);
  run<4, 128, 3, false>("TS  A read from columns the next chain overwrites", G, out, err);
  run<5, 128, 3, false>("TS  same chains, A from columns nobody writes", G, out, err);
  run<6, 128, 3, false>("TS  chains restarted (accumulate off on the first)", G, out, err);
  run<7, 128, 3, false>("TS  two issuing warps, G chains each (per own instr)", G, out, err);
  run<7, 128, 3, true, true>("TS  two issuing warps + 8 math warps", G, out, err);
  run<2, 128, 3, true, true, 1>("TS  8 math warps, dependent smem load / 20 instr", G, out, err);
  run<2, 128, 3, true, true, 2>("TS  8 math warps, nanosleep(0) / 20 instr", G, out, err);
  run<2, 128, 3, true, true, 3>("TS  8 math warps, bar.warp.sync / 20 instr", G, out, err);
  run<2, 128, 3, false, false, 0, true>("TS  warp-uniform issue (elect_one), alone", G, out, err);
  run<2, 128, 3, true, true, 0, true>("TS  warp-uniform issue (elect_one) + 8 math warps", G, out, err);
  run<0, 256, 1, false>("SS  N=256 B K-major, 1 accumulator", G, out, err);
  run<2, 256, 1, false>("TS  N=256 B K-major, 1 accumulator", G, out, err);
  return 0;
}
