"""Autograd-aware hot ops with two implementations each.

``torch_ref`` (plain PyTorch; CPU oracle and CUDA "library" baseline) and the sm_100a extension
(``native.lib()``) share one set of ``torch.autograd.Function`` wrappers, so what is saved for
backward is identical on both paths and is the minimum the backward needs (norm input + rstd,
rotated q/k, attention out + LSE, the gate/up pre-activation).

Tensor conventions: batch size is 1 and folded away, as in the reference
(reference ``utils/linear_tpsp.py:151-154`` views ``[1, s, h]`` as ``[s, h]``); activations are
``[T, features]`` and attention tensors ``[T, heads, head_dim]``.
"""
from __future__ import annotations

import math
import os
from typing import NamedTuple, Optional, Tuple

import torch
from torch.autograd import Function

from . import native, torch_ref as R

# ----------------------------------------------------------------------------- GEMM primitives


class RopeEpilogue(NamedTuple):
    """Rotary embedding folded into the epilogue of a packed q|k|v projection: the output columns are heads in groups
    of ``period_cols`` columns, the first ``rot_cols`` columns of each group (the q and k heads) are rotated with
    ``cos`` / ``sin`` [rows, head_dim / 2] fp32, indexed by output row.  The reference rotates q and k in separate
    passes after the projection (reference ``decoder/odysseus.py:200-226``)."""
    cos: torch.Tensor
    sin: torch.Tensor
    rot_cols: int
    period_cols: int

    def in_kernel(self, n_cols: int) -> bool:
        """The GEMM kernels' epilogue handles head_dim 128 with whole heads per group."""
        return (self.cos.shape[1] == 64 and self.period_cols % 128 == 0 and self.rot_cols % 128 == 0
                and n_cols % self.period_cols == 0)


def rope_grouped_(src: torch.Tensor, dst: torch.Tensor, n_rot: int, period: int, cos, sin, inverse: bool) -> torch.Tensor:
    """src [T, heads, hd] -> dst (may be src): heads in groups of ``period``, the first ``n_rot`` of each rotated and the
    others copied.  One kernel where the reference's block does a copy and a rotation per tensor
    (reference ``decoder/odysseus.py:200-226``)."""
    if native.use_native(src):
        native.lib().rope_grouped_(src, dst, n_rot, period, cos, sin, inverse)
        return dst
    T, heads, hd = src.shape
    g = heads // period
    s4 = src.reshape(T, g, period, hd)
    rot = R.rope_apply(s4[:, :, :n_rot].reshape(T, g * n_rot, hd), cos, sin, inverse).reshape(T, g, n_rot, hd)
    dst.copy_(torch.cat([rot.to(src.dtype), s4[:, :, n_rot:]], dim=2).reshape(T, heads, hd))
    return dst


def apply_rope_epilogue_(y: torch.Tensor, rope: RopeEpilogue) -> torch.Tensor:
    """What the kernels' rotary epilogue computes, as a pass over the finished product y [rows, N] (in place)."""
    hd = 2 * rope.cos.shape[1]
    y3 = y.view(y.shape[0], y.shape[1] // hd, hd)
    rope_grouped_(y3, y3, rope.rot_cols // hd, rope.period_cols // hd, rope.cos, rope.sin, False)
    return y


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, rope: Optional[RopeEpilogue] = None,
            residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[M,N] = A[M,K] @ B[N,K]^T  (the forward of a linear layer: x @ W^T), optionally with the rotary embedding of a
    packed q|k|v projection applied to the product and / or a residual [M, N] added to it, both in the GEMM epilogue."""
    if native.use_native(a):
        lib = native.lib()
        if rope is None or rope.in_kernel(b.shape[0]):
            if rope is None and residual is None:
                return lib.gemm(a, b, out, 0, False)
            return lib.gemm(a, b, out, 0, False, tuple(rope) if rope is not None else None, residual)
        y = apply_rope_epilogue_(lib.gemm(a, b, out, 0, False), rope)       # head_dim other than 128: a pass of its own
        return y if residual is None else y.add_(residual)
    y = a @ b.t() if out is None else torch.matmul(a, b.t(), out=out)
    if rope is not None:
        apply_rope_epilogue_(y, rope)
    if residual is not None:
        y += residual
    return y


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[M,N] = A[M,K] @ B[K,N]  (dgrad: dy @ W)."""
    if native.use_native(a):
        return native.lib().gemm(a, b, out, 1, False)
    if out is None:
        return a @ b
    return torch.matmul(a, b, out=out)


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
            accumulate: bool = False) -> torch.Tensor:
    """C[M,N] (+)= A[K,M]^T @ B[K,N]  (wgrad: dy^T @ x)."""
    if native.use_native(a):
        return native.lib().gemm(a, b, out, 2, accumulate)
    if out is None:
        return a.t() @ b
    if accumulate:
        out.addmm_(a.t(), b)
        return out
    return torch.matmul(a.t(), b, out=out)


def store_weight_grad(w: torch.Tensor, dy2d: torch.Tensor, x2d: torch.Tensor) -> Optional[torch.Tensor]:
    """wgrad ``dy^T @ x`` for weight ``w [out, in]``.

    When the optimizer has attached a flat gradient view ``w.main_grad`` the GEMM writes (or, on a
    second use of the same weight within a step, accumulates) straight into it and autograd gets
    ``None`` - no per-parameter allocation and no extra accumulate pass.  The reference keeps this
    Megatron feature as a dead branch (reference ``utils/linear_tpsp.py:262-289``)."""
    mg = getattr(w, "main_grad", None)
    if mg is None:
        return gemm_tn(dy2d, x2d)
    acc = bool(getattr(w, "_grad_written", False))
    gemm_tn(dy2d, x2d, out=mg, accumulate=acc)
    w._grad_written = True
    return None


def deliver_grad(w: torch.Tensor, g: torch.Tensor) -> Optional[torch.Tensor]:
    """Hand a finished gradient ``g`` (same shape as ``w``) to ``main_grad`` if present."""
    mg = getattr(w, "main_grad", None)
    if mg is None:
        return g.to(w.dtype)
    if getattr(w, "_grad_written", False):
        mg.add_(g.to(mg.dtype))
    else:
        mg.copy_(g)
        w._grad_written = True
    return None


class _Linear(Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm_nt(x2, w)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = gemm_nn(dy2, w).view_as(x) if ctx.needs_input_grad[0] else None
        dw = store_weight_grad(w, dy2, x2) if ctx.needs_input_grad[1] else None
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x @ w^T with w [out, in] (no bias: Llama has none)."""
    return _Linear.apply(x, w)


# ----------------------------------------------------------------------------- RMSNorm


class _RMSNorm(Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        if native.use_native(x):
            y, rstd = native.lib().rmsnorm_fwd(x, w, eps)
        else:
            y, rstd = R.rmsnorm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        if native.use_native(x):
            dx, dw = native.lib().rmsnorm_bwd(dy, x, w, rstd, None)
        else:
            dx, dw = R.rmsnorm_bwd(dy, x, w, rstd)
        return dx, deliver_grad(w, dw), None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return _RMSNorm.apply(x, w, eps)


class _AddRMSNorm(Function):
    """s = x + delta ; y = rmsnorm(s).  Returns (s, y); the residual stream never takes a
    separate elementwise pass (HF Llama does the add as its own kernel)."""

    @staticmethod
    def forward(ctx, x, delta, w, eps):
        if native.use_native(x):
            s, y, rstd = native.lib().add_rmsnorm_fwd(x, delta, w, eps)
        else:
            s, y, rstd = R.add_rmsnorm_fwd(x, delta, w, eps)
        ctx.save_for_backward(s, w, rstd)
        return s, y

    @staticmethod
    def backward(ctx, ds, dy):
        s, w, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        if native.use_native(s):
            dx, dw = native.lib().rmsnorm_bwd(dy, s, w, rstd, ds.contiguous())
        else:
            dx, dw = R.rmsnorm_bwd(dy, s, w, rstd)
            dx = (dx.float() + ds.float()).to(dx.dtype)
        return dx, dx, deliver_grad(w, dw), None


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor, w: torch.Tensor, eps: float):
    return _AddRMSNorm.apply(x, delta, w, eps)


class _RMSNormKeep(Function):
    """y = rmsnorm(s), returning (s, y) with s passed through: the residual stream arrives already summed (the block
    before it added the residual in its GEMM epilogue) and goes on to the next block's epilogue, so its gradient comes
    back as a second input of this op's backward and joins the normalisation's gradient in the same kernel."""

    @staticmethod
    def forward(ctx, s, w, eps):
        if native.use_native(s):
            y, rstd = native.lib().rmsnorm_fwd(s, w, eps)
        else:
            y, rstd = R.rmsnorm_fwd(s, w, eps)
        ctx.save_for_backward(s, w, rstd)
        return s.view_as(s), y

    @staticmethod
    def backward(ctx, ds, dy):
        s, w, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        if native.use_native(s):
            dx, dw = native.lib().rmsnorm_bwd(dy, s, w, rstd, ds.contiguous())
        else:
            dx, dw = R.rmsnorm_bwd(dy, s, w, rstd)
            dx = (dx.float() + ds.float()).to(dx.dtype)
        return dx, deliver_grad(w, dw), None


def rmsnorm_keep(s: torch.Tensor, w: torch.Tensor, eps: float):
    """(s, rmsnorm(s)); see ``_RMSNormKeep``."""
    return _RMSNormKeep.apply(s, w, eps)


# Work folded into GEMM epilogues by the model blocks: "rope" - the q|k|v projection rotates q and k; "residual" - the
# output projections of the attention and MLP blocks add the residual stream.  Switchable for A/B measurements.
_EPILOGUE_FUSION = {"rope": os.environ.get("ODY_FUSE_ROPE", "1") != "0", "residual": os.environ.get("ODY_FUSE_RESIDUAL", "1") != "0"}


def fuse_epilogues(rope: Optional[bool] = None, residual: Optional[bool] = None) -> dict:
    """Set (where not None) and return which epilogue fusions the model blocks use."""
    if rope is not None:
        _EPILOGUE_FUSION["rope"] = bool(rope)
    if residual is not None:
        _EPILOGUE_FUSION["residual"] = bool(residual)
    return dict(_EPILOGUE_FUSION)


def epilogue_fusion(what: str) -> bool:
    return _EPILOGUE_FUSION[what]


# ----------------------------------------------------------------------------- RoPE


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float):
    if native.use_native(positions):
        return native.lib().rope_tables(positions, head_dim, float(theta))
    return R.rope_tables(positions, head_dim, theta)


class _RoPE(Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        if native.use_native(x):
            return native.lib().rope_apply(x.contiguous(), cos, sin, False)
        return R.rope_apply(x, cos, sin, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        if native.use_native(dy):
            return native.lib().rope_apply(dy.contiguous(), cos, sin, True), None, None
        return R.rope_apply(dy, cos, sin, True), None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on [T, H, hd] (HF convention, reference decoder/odysseus.py:210-213)."""
    return _RoPE.apply(x, cos, sin)


# ----------------------------------------------------------------------------- SwiGLU


class _SwiGLU(Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        if native.use_native(gu):
            return native.lib().swiglu_fwd(gu)
        return R.swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dh):
        (gu,) = ctx.saved_tensors
        dh = dh.contiguous()
        if native.use_native(gu):
            return native.lib().swiglu_bwd(dh, gu)
        return R.swiglu_bwd(dh, gu)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2i] = [gate | up] -> silu(gate) * up (reference decoder/odysseus.py:293-295)."""
    return _SwiGLU.apply(gate_up)


# ----------------------------------------------------------------------------- attention


def attn_block_fwd(q, k, v, causal: bool, scale: Optional[float] = None):
    """One attention block -> (out [Tq,H,hd], lse [H,Tq] fp32)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if native.use_native(q) and native.has_native_attention() and q.shape[-1] == 128:
        return native.lib().attn_fwd(q, k, v, causal, scale)
    if q.is_cuda and q.dtype in (torch.bfloat16, torch.float16):
        return _aten_flash_fwd(q, k, v, causal, scale)
    return R.attn_fwd(q, k, v, causal, scale)


def attn_block_bwd(do, q, k, v, o, lse, causal: bool, scale: Optional[float] = None):
    """Backward of one block given the final (o, lse) of q's rows -> (dq, dk, dv)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if native.use_native(q) and native.has_native_attention_bwd() and q.shape[-1] == 128:
        return native.lib().attn_bwd(do, q, k, v, o, lse, causal, scale, None, None, None)
    if q.is_cuda and q.dtype in (torch.bfloat16, torch.float16):
        return _aten_flash_bwd(do, q, k, v, o, lse, causal, scale)
    return R.attn_bwd(do, q, k, v, o, lse, causal, scale)


def _aten_flash_fwd(q, k, v, causal, scale):
    # library path: the FlashAttention-2 kernels bundled with torch, layout [B, T, H, hd]
    out, lse, rng, unused, _ = torch.ops.aten._flash_attention_forward(
        q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), None, None, q.shape[0], k.shape[0],
        0.0, causal, False, scale=scale)
    return out.squeeze(0), lse.squeeze(0)


def _aten_flash_bwd(do, q, k, v, o, lse, causal, scale):
    rng = torch.zeros(2, dtype=torch.uint64, device=q.device)
    dq, dk, dv = torch.ops.aten._flash_attention_backward(
        do.unsqueeze(0).contiguous(), q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), o.unsqueeze(0),
        lse.unsqueeze(0).contiguous(), None, None, q.shape[0], k.shape[0], 0.0, causal, rng,
        torch.zeros((), dtype=torch.int64, device=q.device), scale=scale)
    return dq.squeeze(0), dk.squeeze(0), dv.squeeze(0)


class _Attention(Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = attn_block_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale = causal, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = attn_block_bwd(do.contiguous(), q, k, v, o, lse, ctx.causal, ctx.scale)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              scale: Optional[float] = None) -> torch.Tensor:
    """Softmax attention, q [T,H,hd], k/v [T,Hkv,hd] (GQA when Hkv < H)."""
    return _Attention.apply(q, k, v, causal, scale)


# ----------------------------------------------------------------------------- cross-entropy


class _CrossEntropySum(Function):
    """sum_t CE(logits_t, target_t) * scale, with the gradient written in place over ``logits``
    (the reference uses flash-attn's Triton loss with ``inplace_backward=True``, train.py:173)."""

    @staticmethod
    def forward(ctx, logits, targets, scale, ignore_index):
        if native.use_native(logits):
            loss, lse = native.lib().ce_fwd(logits, targets, ignore_index)
        else:
            loss, lse = R.cross_entropy_fwd(logits, targets, ignore_index)
        ctx.save_for_backward(logits, targets, lse)
        ctx.scale, ctx.ignore_index = scale, ignore_index
        return loss.sum() * scale

    @staticmethod
    def backward(ctx, dloss):
        logits, targets, lse = ctx.saved_tensors
        # dloss is a 0-d tensor; fold it into the scale on the host only when it is the usual 1.0
        scale_t = dloss * ctx.scale
        if native.use_native(logits):
            native.lib().ce_bwd_(logits, targets, lse, scale_t.float().reshape(1), ctx.ignore_index)
        else:
            R.cross_entropy_bwd_(logits, targets, lse, scale_t.float(), ctx.ignore_index)
        return logits, None, None, None


def cross_entropy_sum(logits: torch.Tensor, targets: torch.Tensor, scale: float = 1.0,
                      ignore_index: int = -100) -> torch.Tensor:
    """Summed token cross-entropy times ``scale`` (callers pass 1/global_token_count so every
    rank's partial adds up to the global mean).  ``logits`` is overwritten during backward."""
    return _CrossEntropySum.apply(logits, targets, scale, ignore_index)


class _ChunkedLinearCrossEntropy(Function):
    """lm_head + cross-entropy over row chunks, gradients computed in the same pass.

    ``[t, V]`` logits never exist whole: per chunk of ``chunk_rows`` tokens the logits are formed, reduced to
    loss and log-sum-exp, overwritten in place by their gradient and consumed at once by the two backward GEMMs
    (``dh`` rows; ``dW`` accumulated over chunks).  The ZeRO-3 weight is gathered once for both directions and its
    gradient reduce-scattered once.  Backward only scales the stored gradients by the incoming scalar."""

    @staticmethod
    def forward(ctx, h, w, targets, scale, ignore_index, group, chunk_rows):
        from ..comm import torch_backend as C
        n = C.group_size(group)
        full = C.all_gather_rows(w.detach(), group) if n > 1 else w.detach()
        t, V = h.shape[0], full.shape[0]
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        use_native = native.use_native(h)
        dh = torch.empty_like(h) if need_dh else None
        dw_full = torch.empty_like(full) if need_dw else None
        total = torch.zeros((), dtype=torch.float32, device=h.device)
        scale_t = torch.full((1,), float(scale), dtype=torch.float32, device=h.device)
        first = True
        for r0 in range(0, t, chunk_rows):
            hc, tc = h[r0:r0 + chunk_rows], targets[r0:r0 + chunk_rows]
            logits = gemm_nt(hc, full)
            if use_native:
                loss, lse = native.lib().ce_fwd(logits, tc, ignore_index)
            else:
                loss, lse = R.cross_entropy_fwd(logits, tc, ignore_index)
            total += loss.sum()
            if not (need_dh or need_dw):
                continue
            if use_native:
                native.lib().ce_bwd_(logits, tc, lse, scale_t, ignore_index)
            else:
                R.cross_entropy_bwd_(logits, tc, lse, scale_t[0], ignore_index)
            if need_dh:
                gemm_nn(logits, full, out=dh[r0:r0 + chunk_rows])
            if need_dw:
                gemm_tn(logits, hc, out=dw_full, accumulate=not first)
            first = False
        dw = None
        if need_dw:
            dw = C.reduce_scatter_rows(dw_full, group) if n > 1 else dw_full
        ctx.w = w
        ctx.save_for_backward(*(x for x in (dh, dw) if x is not None))
        ctx.have = (need_dh, need_dw)
        return total * scale

    @staticmethod
    def backward(ctx, dloss):
        saved = list(ctx.saved_tensors)
        dh = saved.pop(0) if ctx.have[0] else None
        dw = saved.pop(0) if ctx.have[1] else None
        if dh is not None:
            dh = dh * dloss.to(dh.dtype)
        gw = deliver_grad(ctx.w, dw * dloss.to(dw.dtype)) if dw is not None else None
        return dh, gw, None, None, None, None, None


def linear_cross_entropy_sum(h: torch.Tensor, w_shard: torch.Tensor, targets: torch.Tensor, scale: float, group,
                             chunk_rows: int, ignore_index: int = -100) -> torch.Tensor:
    """``cross_entropy_sum(h @ gather(w_shard)^T, targets, scale)`` without materialising the logits:
    ``h [t, d]``, ``w_shard [V/n, d]`` (ZeRO-3 over ``group``), evaluated ``chunk_rows`` tokens at a time.
    The reference upcasts the whole ``[L/N, V]`` logits tensor to fp32 before its loss (reference
    ``train.py:210-216`` through HF's ``LlamaForCausalLM``), which is what bounds its sequence length."""
    return _ChunkedLinearCrossEntropy.apply(h, w_shard, targets, scale, ignore_index, group, int(chunk_rows))


# ----------------------------------------------------------------------------- embedding


class _Embedding(Function):
    @staticmethod
    def forward(ctx, ids, w):
        ctx.save_for_backward(ids)
        ctx.w = w
        return w.index_select(0, ids)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        w = ctx.w
        mg = getattr(w, "main_grad", None)
        if mg is not None and not getattr(w, "_grad_written", False):
            mg.zero_()
            mg.index_add_(0, ids, dy.to(mg.dtype))
            w._grad_written = True
            return None, None
        g = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        g.index_add_(0, ids, dy.float())
        return None, deliver_grad(w, g)


def embedding(ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _Embedding.apply(ids, w)
