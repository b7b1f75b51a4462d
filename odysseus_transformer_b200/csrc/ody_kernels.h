// Host-callable launchers of the sm_100a kernels.  Plain pointers and a stream: no torch types, so
// the .cu files build in seconds and can be called from any host runtime.  Every launcher returns a
// cudaError_t-compatible int (0 = success) and never allocates device memory; workspaces are passed in.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- RMSNorm (bf16 activations, fp32 statistics). delta may be null (no residual add).
int ody_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* sum_out, void* y, float* rstd,
                    int64_t rows, int dim, float eps, cudaStream_t stream);
// dx = d(rmsnorm)/dx * dy (+ ds when non-null); dw_partial [ody_rmsnorm_bwd_blocks(), dim] fp32 workspace,
// reduced into dw [dim] fp32 by the same call.
int ody_rmsnorm_bwd_blocks(int64_t rows, int dim);
int ody_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* ds, void* dx,
                    float* dw, float* dw_partial, int64_t rows, int dim, cudaStream_t stream);

// ---- RoPE (rotate-half).  positions int64 [T]; tables fp32 [T, hd/2].
int ody_rope_tables(const int64_t* positions, float* cos_out, float* sin_out, int64_t T, int head_dim, float theta,
                    cudaStream_t stream);
// rotates heads [0, n_rot) of x [T, heads, hd] (row stride in elements) in place; inverse = transpose rotation
int ody_rope_inplace(void* x, const float* cos_t, const float* sin_t, int64_t T, int n_rot, int head_dim,
                     int64_t row_stride, int inverse, cudaStream_t stream);
// general form: heads come in groups of `period`, the first n_rot of each group are rotated; src == dst rotates in place,
// otherwise every head is written to dst (the others copied), so that a copy followed by a rotation is one pass
int ody_rope(const void* src, void* dst, const float* cos_t, const float* sin_t, int64_t T, int heads, int period,
             int n_rot, int head_dim, int64_t src_stride, int64_t dst_stride, int inverse, cudaStream_t stream);

// ---- SwiGLU: gu [T, 2I] = [gate | up]  ->  h [T, I] ; bwd writes dgu [T, 2I]
int ody_swiglu_fwd(const void* gu, void* h, int64_t T, int64_t I, cudaStream_t stream);
int ody_swiglu_bwd(const void* dh, const void* gu, void* dgu, int64_t T, int64_t I, cudaStream_t stream);

// ---- cross-entropy over bf16 logits [T, V]: per-row loss and lse (fp32); bwd overwrites logits with
// (softmax - onehot) * scale[0]  (scale on device), rows with target == ignore_index get 0.
int ody_ce_fwd(const void* logits, const int64_t* targets, float* loss, float* lse, int64_t T, int64_t V,
               int64_t ignore_index, cudaStream_t stream);
int ody_ce_bwd(void* logits, const int64_t* targets, const float* lse, const float* scale, int64_t T, int64_t V,
               int64_t ignore_index, cudaStream_t stream);

// ---- AdamW on flat shards: fp32 master / m / v, bf16 grad in, bf16 param out.  guard (device, may be null):
// when *guard != 0 at run time the kernel changes nothing (a failed step must not reach the master weights).
int ody_adamw(float* master, float* m, float* v, const void* grad, void* param, int64_t n, float lr, float beta1,
              float beta2, float eps, float weight_decay, int step, float grad_scale, const float* guard,
              cudaStream_t stream);

// ---- merge of two partial attention results (ring attention): out/lse fp32 running, o bf16 / l fp32 partial
int ody_attn_merge(float* out, float* lse, const void* o, const float* l, int64_t T, int H, int hd, int64_t row0,
                   int64_t T_total, cudaStream_t stream);
// dst [T, C] bf16 (row pitch dst_ld): rows [begin_i, begin_i + rows_i) += src_i (row pitch src_ld_i), fp32 sum over n <= 8 sources
int ody_sum_rows(void* dst, int64_t dst_ld, int64_t T, int64_t C, const void* const* src, const int64_t* src_ld,
                 const int64_t* begin, const int64_t* rows, int n, cudaStream_t stream);
// one-pass merge of n <= 8 attention partials (o_i [rows_i, H, hd] bf16, lse_i [H, rows_i]) covering rows
// [begin_i, begin_i + rows_i) of out [T, H, hd] bf16 / lse [H, T]; every row must be covered by at least one partial
int ody_attn_merge_parts(void* out, float* lse, int64_t T, int H, int hd, const void* const* o, const float* const* l,
                         const int64_t* begin, const int64_t* rows, int n, cudaStream_t stream);

// ---- bf16 GEMM on tcgen05 (fp32 accumulate in TMEM).  layout 0: C = A[M,K] B[N,K]^T ; 1: C = A[M,K] B[K,N] ;
// 2: C = A[K,M]^T B[K,N].  ld* are row pitches in elements (multiples of 8).  accumulate: C += result.
// err: device int that receives a non-zero code if a bounded wait inside the kernel gave up.
int ody_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                  int layout, int accumulate, int* err, cudaStream_t stream);
// the same GEMM on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles, clusters of two); ody_gemm_bf16 picks between
// the two kernels per problem unless ody_gemm_set_variant(1 = one-CTA only, 2 = pairs only, 0 = automatic) says otherwise
int ody_gemm_bf16_2cta(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                       int layout, int accumulate, int* err, cudaStream_t stream);
int ody_gemm_set_variant(int variant);
// Work folded into the GEMM epilogue (all optional).
//  rope_*: rotary embedding of a packed q|k|v projection with head_dim 128 - output columns in groups of
//    rope_period_cols, the first rope_rot_cols of each group rotated with cos / sin [M, 64] fp32 indexed by output row.
//  residual: bf16 [M, N] (row pitch residual_ld) added to the product; C need not hold it (not together with accumulate).
typedef struct OdyEpilogue {
  const float* rope_cos; const float* rope_sin;
  int rope_period_cols, rope_rot_cols;
  const void* residual; int64_t residual_ld;
} OdyEpilogue;
int ody_gemm_bf16_ex(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                     int layout, int accumulate, const OdyEpilogue* epilogue, int* err, cudaStream_t stream);
int ody_gemm_bf16_2cta_ex(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                          int layout, int accumulate, const OdyEpilogue* epilogue, int* err, cudaStream_t stream);

// ---- attention forward (head_dim 128): q [Tq,H,128], k/v [Tk,Hkv,128], row pitches in elements; out bf16, lse [H,Tq]
// fp32 natural log.  causal needs Tq == Tk.
int ody_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int Tq, int Tk, int H, int Hkv,
                  int64_t q_row, int64_t k_row, int64_t v_row, int64_t o_row, int causal, float scale, int* err,
                  cudaStream_t stream);

// ---- attention backward.  workspace: ody_flash_bwd_workspace_bytes(Tq, H) bytes of scratch, 16-byte aligned.
// dq/dk/dv may be row-pitched views (e.g. slices of one packed gradient tensor).
int64_t ody_flash_bwd_workspace_bytes(int Tq, int H);
/* 1 (default): dK/dV kernel + dQ kernel, no atomics; 0: one fused dK/dV/dQ kernel, dQ summed with fp32 reductions */
int ody_flash_bwd_set_variant(int variant);
/* CTAs of the forward grid (one per 256 query rows and head): the upper bound of a push description's n_cta */
int ody_flash_fwd_ctas(int Tq, int H);
/* 1: the forward keeps its Q / K tiles as eight 32-byte-swizzled slices, 0: as two 128-byte-swizzled halves */
int ody_flash_fwd_set_kslice(int on);
/* development builds (-DODY_ATTN_TRACE) only: [64][16] int64 SM-clock stamps of one forward CTA; otherwise cudaErrorNotSupported */
int ody_flash_fwd_set_trace(long long* buf);
/* optional 96 x 8 int64 timeline of one CTA of each backward kernel; recorded only by a build with -DODY_ATTN_TRACE */
void ody_flash_bwd_set_trace(long long* buf);
int ody_flash_bwd(const void* dO, const void* q, const void* k, const void* v, const void* o, const float* lse, void* dq,
                  void* dk, void* dv, void* workspace, int Tq, int Tk, int H, int Hkv, int64_t do_row, int64_t q_row,
                  int64_t k_row, int64_t v_row, int64_t o_row, int64_t dq_row, int64_t dk_row, int64_t dv_row, int causal,
                  float scale, int* err, cudaStream_t stream);
// full form: with n_split > 0 the gradients go, split by rows of split_rows (a multiple of 128), to dq_split[d] /
// dk_split[d] / dv_split[d] (possibly peer memory; row pitches dq_row / dk_row / dv_row) instead of dq / dk / dv
int ody_flash_bwd_ex(const void* dO, const void* q, const void* k, const void* v, const void* o, const float* lse, void* dq,
                     void* dk, void* dv, void* workspace, int Tq, int Tk, int H, int Hkv, int64_t do_row, int64_t q_row,
                     int64_t k_row, int64_t v_row, int64_t o_row, int64_t dq_row, int64_t dk_row, int64_t dv_row, int causal,
                     float scale, void* const* dq_split, void* const* dk_split, void* const* dv_split, int n_split,
                     int split_rows, int* err, cudaStream_t stream);

// ---- GEMM fused with an all-gather of one operand and/or a reduce-scatter of the result over peer memory
// (gemm_comm.cu).  Descriptions are plain data; pointers in *_peer[p] address rank p's symmetric memory.
typedef struct OdyGatherDesc {
  const void* shard; int64_t shard_ld;
  void* gathered_peer[8]; uint32_t* flags_peer[8]; uint32_t* counters_peer[8]; uint32_t* free_peer[8];
  uint32_t* gemm_done;
  void* stats;           /* optional [n_cta][4] uint64 ns: comm begin, comm end, producer row-wait time, CTA end */
  int n_ranks, rank, chunk_rows, cols;
  int n_cta;             /* CTAs of this launch = min(tiles, SMs); checked against the launcher's grid */
  uint32_t push_total;   /* running total of CTAs that pushed into this slot (all uses, the current one included) */
  uint32_t consume_total;/* running total of CTAs that consumed this slot (all uses, the current one included) */
  uint32_t epoch, prev_epoch, uses;
  int which;
  int dest_first, dest_count; /* push only: destinations rank + dest_first ... (mod n_ranks); dest_count 0 = every rank, own included */
} OdyGatherDesc;
typedef struct OdyScatterDesc {
  void* stage_peer[8]; uint32_t* arrived_peer[8]; uint32_t* consumed_peer[8];
  uint32_t* reduce_counter; void* out; int64_t out_ld;
  int n_ranks, rank, chunk_rows;
  uint32_t epoch, prev_epoch, arrived_target, uses;
  /* mode 2 = all-to-all on columns (no reduction): column group o of row r -> stage_peer[o][(a2a_row0 + r) * a2a_ld + a2a_col0 + c'] */
  int mode, a2a_cols;
  int64_t a2a_ld, a2a_row0, a2a_col0;
} OdyScatterDesc;
int ody_gemm_comm(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                  int layout, const OdyGatherDesc* gather, const OdyGatherDesc* push, const OdyScatterDesc* scatter, int* err,
                  cudaStream_t stream);
// epilogue: rotary embedding in the epilogues that write whole rows (no scatter, or the all-to-all); the residual in
// the plain epilogue ([M, N]) or in the reduction of the reduce-scatter (this rank's [chunk_rows, N] rows)
int ody_gemm_comm_ex(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                     int layout, const OdyGatherDesc* gather, const OdyGatherDesc* push, const OdyScatterDesc* scatter,
                     const OdyEpilogue* epilogue, int* err, cudaStream_t stream);
int ody_push_shard(const OdyGatherDesc* push, int* err, cudaStream_t stream);
// one-thread kernel: bounded wait until source `src`'s whole shard of the slot's current epoch has arrived here
int ody_wait_shard(const OdyGatherDesc* slot, int src, int* err, cudaStream_t stream);
// tell every pusher that this rank has finished reading the slot's current epoch (stream-ordered after the readers)
int ody_signal_free(const OdyGatherDesc* slot, cudaStream_t stream);
// n <= 32 threads: thread i with bit i of mask set waits (bounded) until base[i] >= target
int ody_wait_flags(const uint32_t* base, uint32_t mask, uint32_t target, int* err, cudaStream_t stream);
// for every p with bit p of mask set: ptrs[p][index] <- value with release at system scope, after a system fence
int ody_signal_flags(uint32_t* const* ptrs, int n, uint32_t mask, int index, uint32_t value, cudaStream_t stream);
// attention forward whose comm warps also push a K/V shard to ring peers (push == NULL: plain ody_flash_fwd)
int ody_flash_fwd_push(const void* q, const void* k, const void* v, void* o, float* lse, int Tq, int Tk, int H, int Hkv,
                       int64_t q_row, int64_t k_row, int64_t v_row, int64_t o_row, int causal, float scale,
                       const OdyGatherDesc* push, int* err, cudaStream_t stream);
// full form: optional push, and optional extra destinations for the output rows (Ulysses head->sequence exchange):
// rows [d * split_rows, (d + 1) * split_rows) are also stored to o_split[d] ([split_rows, H, 128], row pitch split_row)
int ody_flash_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse, int Tq, int Tk, int H, int Hkv,
                     int64_t q_row, int64_t k_row, int64_t v_row, int64_t o_row, int causal, float scale,
                     const OdyGatherDesc* push, void* const* o_split, int n_split, int split_rows, int64_t split_row, int* err,
                     cudaStream_t stream);
int ody_flash_set_peer_wait_limit(long long cycles);
int ody_flash_set_push_order(int unit_major);
// schedule of the comm warps' pushes on the current device: 0 destination by destination (default), 1 every unit to all
// destinations at once
int ody_set_push_order(int unit_major);
// bound (SM clock cycles) of every wait inside the fused kernels on the current device; default ~10 s
int ody_set_peer_wait_limit(long long cycles);

// running totals (ns) of the time the fused kernels of the current device spend waiting on other GPUs; see gemm_comm.cu
int ody_set_wait_accumulator(unsigned long long* acc);


#ifdef __cplusplus
}
#endif
