// Memory-bound hot ops for sm_100a: RMSNorm(+residual) fwd/bwd, RoPE, SwiGLU fwd/bwd, cross-entropy
// fwd / in-place bwd, fused AdamW over flat shards, attention partial-result merge.
//
// The reference gets these from unfused ATen elementwise kernels inside HF Llama, a Triton loss from
// flash-attn and torch.optim.AdamW (reference train.py:167,173; decoder/odysseus.py:210-213,293-295).
// Every kernel here moves 16 bytes per thread per access and touches each operand once.
#include <string.h>

#include "common.cuh"
#include "ody_kernels.h"

namespace ody {

// ------------------------------------------------------------------------------------------- RMSNorm

template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_fwd_k(const bf16* __restrict__ x, const bf16* __restrict__ delta,
                                                     const bf16* __restrict__ w, bf16* __restrict__ sum_out,
                                                     bf16* __restrict__ y, float* __restrict__ rstd, int dim,
                                                     float eps) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const bf16* xr = x + row * dim;
  float vals[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 8;
    if (c < dim) {
      bf16x8 p = ld8(xr + c);
      if (delta != nullptr) {
        float a[8], b[8];
        unpack8(p, a);
        unpack8(ld8(delta + row * dim + c), b);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] += b[j];
        p = pack8(a);  // the residual stream is stored in bf16; the norm sees the stored value
        st8(sum_out + row * dim + c, p);
      }
      unpack8(p, vals[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
    }
  }
  ss = block_sum(ss, red);
  const float rs = rsqrtf(ss / (float)dim + eps);
  if (threadIdx.x == 0) rstd[row] = rs;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 8;
    if (c < dim) {
      float wv[8], o[8];
      unpack8(ld8(w + c), wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rs * wv[j];
      st8(y + row * dim + c, pack8(o));
    }
  }
}

// Two rows per loop iteration and one barrier per iteration (the warps' partial dot products go through a
// double-buffered shared array that every thread sums itself).  The kernel is bound by memory latency, so what matters
// is how many row loads are in flight per SM: the rows stay in registers as packed bf16 and are unpacked a second time
// for the output instead of being kept as fp32, which halves the registers and lets two blocks share an SM (with the
// fp32 copies it was one block per SM and a third of the copy bandwidth).
template <int NV>
__global__ void __launch_bounds__(256, NV <= 2 ? 2 : 1) rmsnorm_bwd_k(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                     const bf16* __restrict__ w, const float* __restrict__ rstd,
                                                     const bf16* __restrict__ ds, bf16* __restrict__ dx,
                                                     float* __restrict__ dw_partial, int64_t rows, int dim) {
  constexpr int R = NV <= 2 ? 2 : 1;      // wider rows would spill
  __shared__ __align__(16) float red[2][R][8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float wv[NV][8], acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    if (c < dim) unpack8(ld8(w + c), wv[i]);
  }
  const float inv_dim = 1.f / (float)dim;
  int par = 0;
  for (int64_t row0 = (int64_t)blockIdx.x * R; row0 < rows; row0 += (int64_t)gridDim.x * R, par ^= 1) {
    float rs[R], dot[R];
    bf16x8 pa[R][NV], px[R][NV];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = row0 + r;
      rs[r] = row < rows ? rstd[row] : 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = (threadIdx.x + i * blockDim.x) * 8;
        if (c < dim && row < rows) {
          pa[r][i] = ld8(dy + row * dim + c);
          px[r][i] = ld8(x + row * dim + c);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      dot[r] = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = (threadIdx.x + i * blockDim.x) * 8;
        if (c < dim && row0 + r < rows) {
          float a[8], xh[8];
          unpack8(pa[r][i], a);
          unpack8(px[r][i], xh);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            xh[j] *= rs[r];
            acc[i][j] += a[j] * xh[j];
            dot[r] += a[j] * wv[i][j] * xh[j];
          }
        }
      }
      dot[r] = warp_sum(dot[r]);
      if (lane == 0) red[par][r][wid] = dot[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float4 lo = *reinterpret_cast<const float4*>(&red[par][r][0]), hi = *reinterpret_cast<const float4*>(&red[par][r][4]);
      dot[r] = ((lo.x + lo.y) + (lo.z + lo.w) + (hi.x + hi.y) + (hi.z + hi.w)) * inv_dim;
      const int64_t row = row0 + r;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = (threadIdx.x + i * blockDim.x) * 8;
        if (c < dim && row < rows) {
          float a[8], xh[8], o[8];
          unpack8(pa[r][i], a);
          unpack8(px[r][i], xh);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (a[j] * wv[i][j] - xh[j] * rs[r] * dot[r]) * rs[r];
          if (ds != nullptr) {
            float s[8];
            unpack8(ld8(ds + row * dim + c), s);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += s[j];
          }
          st8(dx + row * dim + c, pack8(o));
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (threadIdx.x + i * blockDim.x) * 8;
    if (c < dim) {
      float* p = dw_partial + (int64_t)blockIdx.x * dim + c;
      *reinterpret_cast<float4*>(p) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
  }
}

// out[c] = sum over the nblocks rows of partial[nblocks, dim].  Block = 32 columns x 8 row slices, so the grid has
// dim / 32 blocks (not dim / 256, which left most SMs idle while a few walked all rows one after the other).
__global__ void __launch_bounds__(256) colsum_k(const float* __restrict__ partial, float* __restrict__ out, int nblocks, int dim) {
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (c < dim) {
    int b = slice;
    for (; b + 24 < nblocks; b += 32) {
      s0 += partial[(int64_t)b * dim + c];
      s1 += partial[(int64_t)(b + 8) * dim + c];
      s2 += partial[(int64_t)(b + 16) * dim + c];
      s3 += partial[(int64_t)(b + 24) * dim + c];
    }
    for (; b < nblocks; b += 8) s0 += partial[(int64_t)b * dim + c];
  }
  red[slice][cx] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (slice == 0 && c < dim) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red[i][cx];
    out[c] = s;
  }
}

// ------------------------------------------------------------------------------------------- RoPE

__global__ void rope_tables_k(const int64_t* __restrict__ pos, float* __restrict__ cos_o, float* __restrict__ sin_o,
                              int64_t T, int half, float theta) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  const int k = (int)(i % half);
  const int64_t t = i / half;
  const float inv_freq = 1.0f / powf(theta, (float)(2 * k) / (float)(2 * half));
  const float ang = (float)pos[t] * inv_freq;
  float s, c;
  sincosf(ang, &s, &c);
  cos_o[i] = c;
  sin_o[i] = s;
}

// Rotary embedding over a [T, heads, head_dim] tensor whose heads come in groups of `period`: the first `n_rot` heads of
// every group are rotated, the rest are not.  In place (COPY false: only the rotated heads are touched) or from `src`
// to `dst` (COPY true: the other heads are copied as they are, so a rotation that follows a copy costs one pass, not two).
template <bool COPY>
__global__ void rope_k(const bf16* __restrict__ src, bf16* __restrict__ dst, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, int64_t T, int groups, int period, int n_rot, int head_dim,
                       int64_t src_stride, int64_t dst_stride, int inverse) {
  const int half = head_dim >> 1;
  const int vec_per_head = half >> 3;
  const int per_group = COPY ? period : n_rot;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = T * groups * per_group * vec_per_head;
  if (i >= total) return;
  const int kv = (int)(i % vec_per_head);
  const int hh = (int)((i / vec_per_head) % ((int64_t)groups * per_group));
  const int64_t t = i / ((int64_t)vec_per_head * groups * per_group);
  const int g = hh / per_group, hg = hh - g * per_group;
  const int64_t col = ((int64_t)g * period + hg) * head_dim + kv * 8;
  const bf16* s1 = src + t * src_stride + col;
  bf16* d1 = dst + t * dst_stride + col;
  if (COPY && hg >= n_rot) {
    st8(d1, ld8(s1));
    st8(d1 + half, ld8(s1 + half));
    return;
  }
  float a[8], b[8], o1[8], o2[8];
  unpack8(ld8(s1), a);
  unpack8(ld8(s1 + half), b);
  const float* cp = cos_t + t * half + kv * 8;
  const float* sp = sin_t + t * half + kv * 8;
  const float4 c0 = *reinterpret_cast<const float4*>(cp), c1 = *reinterpret_cast<const float4*>(cp + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(sp), s1v = *reinterpret_cast<const float4*>(sp + 4);
  const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1v.x, s1v.y, s1v.z, s1v.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float sj = inverse ? -s[j] : s[j];
    o1[j] = a[j] * c[j] - b[j] * sj;
    o2[j] = b[j] * c[j] + a[j] * sj;
  }
  st8(d1, pack8(o1));
  st8(d1 + half, pack8(o2));
}

// ------------------------------------------------------------------------------------------- SwiGLU

__global__ void swiglu_fwd_k(const bf16* __restrict__ gu, bf16* __restrict__ h, int64_t T, int64_t I) {
  const int64_t vpr = I >> 3;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * vpr) return;
  const int64_t t = i / vpr, c = (i % vpr) * 8;
  float g[8], u[8], o[8];
  unpack8(ld8(gu + t * 2 * I + c), g);
  unpack8(ld8(gu + t * 2 * I + I + c), u);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
  st8(h + t * I + c, pack8(o));
}

__global__ void swiglu_bwd_k(const bf16* __restrict__ dh, const bf16* __restrict__ gu, bf16* __restrict__ dgu,
                             int64_t T, int64_t I) {
  const int64_t vpr = I >> 3;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * vpr) return;
  const int64_t t = i / vpr, c = (i % vpr) * 8;
  float g[8], u[8], d[8], dg[8], du[8];
  unpack8(ld8(gu + t * 2 * I + c), g);
  unpack8(ld8(gu + t * 2 * I + I + c), u);
  unpack8(ld8(dh + t * I + c), d);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float sig = 1.f / (1.f + __expf(-g[j]));
    dg[j] = d[j] * u[j] * sig * (1.f + g[j] * (1.f - sig));
    du[j] = d[j] * g[j] * sig;
  }
  st8(dgu + t * 2 * I + c, pack8(dg));
  st8(dgu + t * 2 * I + I + c, pack8(du));
}

// ------------------------------------------------------------------------------------------- cross-entropy

__global__ void __launch_bounds__(512) ce_fwd_k(const bf16* __restrict__ logits, const int64_t* __restrict__ targets,
                                                float* __restrict__ loss, float* __restrict__ lse, int64_t V,
                                                int64_t ignore_index) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const bf16* lr = logits + row * V;
  float m = -INFINITY, s = 0.f;
  for (int64_t c = (int64_t)threadIdx.x * 8; c < V; c += (int64_t)blockDim.x * 8) {
    float f[8];
    unpack8(ld8(lr + c), f);
    float mx = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) mx = fmaxf(mx, f[j]);
    const float mn = fmaxf(m, mx);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - mn);
    s = s * __expf(m - mn) + acc;
    m = mn;
  }
  const float M = block_max(m, red);
  const float S = block_sum(s * __expf(m - M), red);
  if (threadIdx.x == 0) {
    const float l = M + logf(S);
    lse[row] = l;
    const int64_t tg = targets[row];
    loss[row] = (tg == ignore_index) ? 0.f : l - __bfloat162float(lr[tg]);
  }
}

__global__ void ce_bwd_k(bf16* __restrict__ logits, const int64_t* __restrict__ targets, const float* __restrict__ lse,
                         const float* __restrict__ scale, int64_t V, int64_t ignore_index) {
  const int64_t row = blockIdx.y;
  const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= V) return;
  const int64_t tg = targets[row];
  const float sc = (tg == ignore_index) ? 0.f : scale[0];
  const float l = lse[row];
  bf16* p = logits + row * V + c;
  float f[8];
  unpack8(ld8(p), f);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float pr = __expf(f[j] - l);
    if (c + j == tg) pr -= 1.f;
    f[j] = pr * sc;
  }
  st8(p, pack8(f));
}

// ------------------------------------------------------------------------------------------- AdamW

__global__ void adamw_k(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                        const bf16* __restrict__ grad, bf16* __restrict__ param, int64_t n, float decay, float beta1,
                        float beta2, float step_size, float inv_sqrt_bc2, float eps, float grad_scale,
                        const float* __restrict__ guard) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  // a non-zero guard word (the step's kernel status, summed over ranks) means some gradient is incomplete:
  // leave master, moments and parameters untouched so the host can stop or restart from here
  if (guard != nullptr && *guard != 0.f) return;
  float g[8];
  unpack8(ld8(grad + i), g);
  float4 w0 = *reinterpret_cast<float4*>(master + i), w1 = *reinterpret_cast<float4*>(master + i + 4);
  float4 m0 = *reinterpret_cast<float4*>(m + i), m1 = *reinterpret_cast<float4*>(m + i + 4);
  float4 v0 = *reinterpret_cast<float4*>(v + i), v1 = *reinterpret_cast<float4*>(v + i + 4);
  float W[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
  float M[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
  float Vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float gj = g[j] * grad_scale;
    M[j] = beta1 * M[j] + (1.f - beta1) * gj;
    Vv[j] = beta2 * Vv[j] + (1.f - beta2) * gj * gj;
    const float denom = sqrtf(Vv[j]) * inv_sqrt_bc2 + eps;
    W[j] = W[j] * decay - step_size * M[j] / denom;
  }
  *reinterpret_cast<float4*>(master + i) = make_float4(W[0], W[1], W[2], W[3]);
  *reinterpret_cast<float4*>(master + i + 4) = make_float4(W[4], W[5], W[6], W[7]);
  *reinterpret_cast<float4*>(m + i) = make_float4(M[0], M[1], M[2], M[3]);
  *reinterpret_cast<float4*>(m + i + 4) = make_float4(M[4], M[5], M[6], M[7]);
  *reinterpret_cast<float4*>(v + i) = make_float4(Vv[0], Vv[1], Vv[2], Vv[3]);
  *reinterpret_cast<float4*>(v + i + 4) = make_float4(Vv[4], Vv[5], Vv[6], Vv[7]);
  st8(param + i, pack8(W));
}

// ------------------------------------------------------------------------------------------- attention merge

// out [T_total, H, hd] fp32 and lse [H, T_total] fp32 are the running result; (o [T, H, hd] bf16,
// l [H, T] fp32) is a partial over a disjoint key set for rows [row0, row0 + T).
__global__ void attn_merge_k(float* __restrict__ out, float* __restrict__ lse, const bf16* __restrict__ o,
                             const float* __restrict__ l, int64_t T, int H, int hd, int64_t row0, int64_t T_total) {
  const int vph = hd >> 3;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = i < T * H * vph;
  float la = 0.f, lb = 0.f;
  int64_t t = 0;
  int h = 0, kv = 0;
  if (live) {
    kv = (int)(i % vph);
    h = (int)((i / vph) % H);
    t = i / ((int64_t)vph * H);
    la = lse[(int64_t)h * T_total + row0 + t];
    lb = l[(int64_t)h * T + t];
  }
  __syncwarp();  // every lane of a (t, h) group has read the old lse before its leader overwrites it
  if (!live) return;
  const float mx = fmaxf(la, lb);
  const float ln = mx + logf(__expf(la - mx) + __expf(lb - mx));
  const float wa = __expf(la - ln), wb = __expf(lb - ln);
  float* po = out + ((row0 + t) * H + h) * hd + kv * 8;
  float b[8];
  unpack8(ld8(o + (t * H + h) * hd + kv * 8), b);
  float4 a0 = *reinterpret_cast<float4*>(po), a1 = *reinterpret_cast<float4*>(po + 4);
  a0 = make_float4(a0.x * wa + b[0] * wb, a0.y * wa + b[1] * wb, a0.z * wa + b[2] * wb, a0.w * wa + b[3] * wb);
  a1 = make_float4(a1.x * wa + b[4] * wb, a1.y * wa + b[5] * wb, a1.z * wa + b[6] * wb, a1.w * wa + b[7] * wb);
  *reinterpret_cast<float4*>(po) = a0;
  *reinterpret_cast<float4*>(po + 4) = a1;
  if (kv == 0) lse[(int64_t)h * T_total + row0 + t] = ln;
}

// dst rows [begin_i, begin_i + rows_i) += src_i, summed in fp32 over all sources; dst [T, C] with row pitch dst_ld.
struct SumRowsArgs {
  const bf16* src[8];
  int64_t src_ld[8], begin[8], rows[8];
  int n;
};
__global__ void sum_rows_k(bf16* __restrict__ dst, int64_t dst_ld, int64_t T, int64_t C, const __grid_constant__ SumRowsArgs a) {
  const int64_t vpr = C >> 3;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * vpr) return;
  const int64_t t = i / vpr, c = (i % vpr) * 8;
  bf16x8 part[8];
  bool on[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    on[k] = k < a.n && t >= a.begin[k] && t < a.begin[k] + a.rows[k];
    if (on[k]) part[k] = ld8(a.src[k] + (t - a.begin[k]) * a.src_ld[k] + c);
  }
  float acc[8];
  unpack8(ld8(dst + t * dst_ld + c), acc);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (on[k]) {
      float b[8];
      unpack8(part[k], b);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += b[e];
    }
  }
  st8(dst + t * dst_ld + c, pack8(acc));
}

// One-pass merge of up to 8 attention partials over disjoint key sets: partial i covers rows
// [begin_i, begin_i + rows_i) with o_i [rows_i, H, hd] bf16 and lse_i [H, rows_i].  out [T, H, hd] bf16, lse [H, T].
struct MergeArgs {
  const bf16* o[8];
  const float* lse[8];
  int64_t begin[8], rows[8];
  int n;
};
__global__ void attn_merge_parts_k(bf16* __restrict__ out, float* __restrict__ lse, int64_t T, int H, int hd,
                                   const __grid_constant__ MergeArgs a) {
  const int vph = hd >> 3;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * H * vph) return;
  const int kv = (int)(i % vph);
  const int h = (int)((i / vph) % H);
  const int64_t t = i / ((int64_t)vph * H);
  float l[8], mx = -INFINITY;
  bf16x8 part[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const bool on = k < a.n && t >= a.begin[k] && t < a.begin[k] + a.rows[k];
    l[k] = -INFINITY;
    if (on) {
      const int64_t tt = t - a.begin[k];
      l[k] = a.lse[k][(int64_t)h * a.rows[k] + tt];
      part[k] = ld8(a.o[k] + (tt * H + h) * hd + kv * 8);
      mx = fmaxf(mx, l[k]);
    }
  }
  float den = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (l[k] != -INFINITY) {
      const float w = __expf(l[k] - mx);
      den += w;
      float b[8];
      unpack8(part[k], b);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += w * b[e];
    }
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] *= inv;
  st8(out + (t * H + h) * hd + kv * 8, pack8(acc));
  if (kv == 0) lse[(int64_t)h * T + t] = den > 0.f ? mx + logf(den) : -INFINITY;
}

}  // namespace ody

// =========================================================================================== launchers

using namespace ody;

static inline int last_err() { return (int)cudaGetLastError(); }
static inline unsigned blocks_for(int64_t n, int per) { return (unsigned)((n + per - 1) / per); }

extern "C" int ody_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* sum_out, void* y, float* rstd,
                               int64_t rows, int dim, float eps, cudaStream_t st) {
  if (dim % 8 != 0 || dim > 256 * 8 * 8) return (int)cudaErrorInvalidValue;
  if (rows == 0) return 0;
  const int nv = (dim + 2047) / 2048;
#define L(NV)                                                                                               \
  rmsnorm_fwd_k<NV><<<(unsigned)rows, 256, 0, st>>>((const bf16*)x, (const bf16*)delta, (const bf16*)w,    \
                                                    (bf16*)sum_out, (bf16*)y, rstd, dim, eps)
  if (nv <= 1) L(1); else if (nv <= 2) L(2); else if (nv <= 4) L(4); else L(8);
#undef L
  return last_err();
}

extern "C" int ody_rmsnorm_bwd_blocks(int64_t rows, int dim) {
  (void)dim;
  int64_t b = 148 * 2;       // two resident blocks per SM (112 registers x 256 threads each)
  return (int)(rows < b ? (rows > 0 ? rows : 1) : b);
}

extern "C" int ody_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* ds,
                               void* dx, float* dw, float* dw_partial, int64_t rows, int dim, cudaStream_t st) {
  if (dim % 8 != 0 || dim > 256 * 8 * 8) return (int)cudaErrorInvalidValue;
  const int nb = ody_rmsnorm_bwd_blocks(rows, dim);
  const int nv = (dim + 2047) / 2048;
#define L(NV)                                                                                                  \
  rmsnorm_bwd_k<NV><<<nb, 256, 0, st>>>((const bf16*)dy, (const bf16*)x, (const bf16*)w, rstd, (const bf16*)ds, \
                                        (bf16*)dx, dw_partial, rows, dim)
  if (nv <= 1) L(1); else if (nv <= 2) L(2); else if (nv <= 4) L(4); else L(8);
#undef L
  colsum_k<<<blocks_for(dim, 32), 256, 0, st>>>(dw_partial, dw, nb, dim);
  return last_err();
}

extern "C" int ody_rope_tables(const int64_t* positions, float* cos_out, float* sin_out, int64_t T, int head_dim,
                               float theta, cudaStream_t st) {
  const int half = head_dim / 2;
  if (T == 0) return 0;
  rope_tables_k<<<blocks_for(T * half, 256), 256, 0, st>>>(positions, cos_out, sin_out, T, half, theta);
  return last_err();
}

extern "C" int ody_rope(const void* src, void* dst, const float* cos_t, const float* sin_t, int64_t T, int heads,
                        int period, int n_rot, int head_dim, int64_t src_stride, int64_t dst_stride, int inverse,
                        cudaStream_t st) {
  if (head_dim % 16 != 0 || src_stride % 8 != 0 || dst_stride % 8 != 0 || period <= 0 || heads % period != 0 ||
      n_rot < 0 || n_rot > period)
    return (int)cudaErrorInvalidValue;
  const int groups = heads / period;
  const bool copy = src != (const void*)dst;
  const int64_t total = T * groups * (copy ? period : n_rot) * (head_dim / 16);
  if (total == 0) return 0;
  if (copy)
    rope_k<true><<<blocks_for(total, 256), 256, 0, st>>>((const bf16*)src, (bf16*)dst, cos_t, sin_t, T, groups, period,
                                                         n_rot, head_dim, src_stride, dst_stride, inverse);
  else
    rope_k<false><<<blocks_for(total, 256), 256, 0, st>>>((const bf16*)src, (bf16*)dst, cos_t, sin_t, T, groups, period,
                                                          n_rot, head_dim, src_stride, dst_stride, inverse);
  return last_err();
}

extern "C" int ody_rope_inplace(void* x, const float* cos_t, const float* sin_t, int64_t T, int n_rot, int head_dim,
                                int64_t row_stride, int inverse, cudaStream_t st) {
  if (n_rot == 0 || T == 0) return 0;
  return ody_rope(x, x, cos_t, sin_t, T, n_rot, n_rot, n_rot, head_dim, row_stride, row_stride, inverse, st);
}

extern "C" int ody_swiglu_fwd(const void* gu, void* h, int64_t T, int64_t I, cudaStream_t st) {
  if (I % 8 != 0) return (int)cudaErrorInvalidValue;
  if (T * I == 0) return 0;
  swiglu_fwd_k<<<blocks_for(T * (I / 8), 256), 256, 0, st>>>((const bf16*)gu, (bf16*)h, T, I);
  return last_err();
}

extern "C" int ody_swiglu_bwd(const void* dh, const void* gu, void* dgu, int64_t T, int64_t I, cudaStream_t st) {
  if (I % 8 != 0) return (int)cudaErrorInvalidValue;
  if (T * I == 0) return 0;
  swiglu_bwd_k<<<blocks_for(T * (I / 8), 256), 256, 0, st>>>((const bf16*)dh, (const bf16*)gu, (bf16*)dgu, T, I);
  return last_err();
}

extern "C" int ody_ce_fwd(const void* logits, const int64_t* targets, float* loss, float* lse, int64_t T, int64_t V,
                          int64_t ignore_index, cudaStream_t st) {
  if (V % 8 != 0) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  ce_fwd_k<<<(unsigned)T, 512, 0, st>>>((const bf16*)logits, targets, loss, lse, V, ignore_index);
  return last_err();
}

extern "C" int ody_ce_bwd(void* logits, const int64_t* targets, const float* lse, const float* scale, int64_t T,
                          int64_t V, int64_t ignore_index, cudaStream_t st) {
  if (V % 8 != 0 || T > 65535) return (int)cudaErrorInvalidValue;
  if (T == 0) return 0;
  dim3 grid(blocks_for(V / 8, 256), (unsigned)T);
  ce_bwd_k<<<grid, 256, 0, st>>>((bf16*)logits, targets, lse, scale, V, ignore_index);
  return last_err();
}

extern "C" int ody_adamw(float* master, float* m, float* v, const void* grad, void* param, int64_t n, float lr,
                         float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale,
                         const float* guard, cudaStream_t st) {
  if (n % 8 != 0) return (int)cudaErrorInvalidValue;
  if (n == 0) return 0;
  const double bc1 = 1.0 - pow((double)beta1, (double)step);
  const double bc2 = 1.0 - pow((double)beta2, (double)step);
  adamw_k<<<blocks_for(n / 8, 256), 256, 0, st>>>(master, m, v, (const bf16*)grad, (bf16*)param, n,
                                                  1.f - lr * weight_decay, beta1, beta2, (float)(lr / bc1),
                                                  (float)(1.0 / sqrt(bc2)), eps, grad_scale, guard);
  return last_err();
}

extern "C" int ody_attn_merge(float* out, float* lse, const void* o, const float* l, int64_t T, int H, int hd,
                              int64_t row0, int64_t T_total, cudaStream_t st) {
  if (hd % 8 != 0 || 32 % (hd / 8) != 0) return (int)cudaErrorInvalidValue;
  const int64_t total = T * H * (hd / 8);
  if (total == 0) return 0;
  attn_merge_k<<<blocks_for(total, 256), 256, 0, st>>>(out, lse, (const bf16*)o, l, T, H, hd, row0, T_total);
  return last_err();
}

extern "C" int ody_sum_rows(void* dst, int64_t dst_ld, int64_t T, int64_t C, const void* const* src, const int64_t* src_ld,
                            const int64_t* begin, const int64_t* rows, int n, cudaStream_t st) {
  if (n < 0 || n > 8 || (C % 8) || (dst_ld % 8) || ((uintptr_t)dst & 15)) return (int)cudaErrorInvalidValue;
  if (n == 0 || T * C == 0) return 0;
  SumRowsArgs a;
  memset(&a, 0, sizeof(a));
  a.n = n;
  for (int k = 0; k < n; ++k) {
    if ((src_ld[k] % 8) || ((uintptr_t)src[k] & 15) || begin[k] < 0 || begin[k] + rows[k] > T) return (int)cudaErrorInvalidValue;
    a.src[k] = (const bf16*)src[k]; a.src_ld[k] = src_ld[k]; a.begin[k] = begin[k]; a.rows[k] = rows[k];
  }
  sum_rows_k<<<blocks_for(T * (C / 8), 256), 256, 0, st>>>((bf16*)dst, dst_ld, T, C, a);
  return last_err();
}

extern "C" int ody_attn_merge_parts(void* out, float* lse, int64_t T, int H, int hd, const void* const* o,
                                    const float* const* l, const int64_t* begin, const int64_t* rows, int n, cudaStream_t st) {
  if (n < 1 || n > 8 || hd % 8 != 0) return (int)cudaErrorInvalidValue;
  if (T * H == 0) return 0;
  MergeArgs a;
  memset(&a, 0, sizeof(a));
  a.n = n;
  for (int k = 0; k < n; ++k) {
    if (begin[k] < 0 || begin[k] + rows[k] > T || ((uintptr_t)o[k] & 15)) return (int)cudaErrorInvalidValue;
    a.o[k] = (const bf16*)o[k]; a.lse[k] = l[k]; a.begin[k] = begin[k]; a.rows[k] = rows[k];
  }
  attn_merge_parts_k<<<blocks_for(T * H * (hd / 8), 256), 256, 0, st>>>((bf16*)out, lse, T, H, hd, a);
  return last_err();
}
