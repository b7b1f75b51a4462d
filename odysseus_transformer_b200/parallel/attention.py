"""Sequence-parallel attention primitives: packed RoPE + causal attention, the Ulysses seq<->head
all-to-all, and zigzag ring attention.

The reference delegates these to dependencies: HF ``apply_rotary_pos_emb`` + flash-attn
(reference ``decoder/odysseus.py:200-263``), ``yunchang.UlyssesAttention`` (called at reference
``decoder/ulysses.py:40-47``) and ``ring_flash_attn.zigzag_ring_flash_attn_func`` (called at
reference ``decoder/ring.py:30-37``).  Here they are written against this package's attention block
primitive ``ops.functional.attn_block_fwd / attn_block_bwd`` so they run on CPU (oracle), on the
library path, and on the sm_100a kernels alike, and they take explicit process groups so they
compose into the inner x ring hybrid.

One core serves every mode: a *packed* ``[Tb, hq + 2 hkv, hd]`` tensor (this rank's query heads, key
heads, value heads, for every token of its ring block) is rotated in place, attended, and its
gradient comes back packed - there are no per-slice copies, transposes or zero-fills around the
attention kernel, and backward keeps exactly one copy of q/k/v.

Ring attention is *pull*-based: NVSwitch gives every GPU full bandwidth to every peer, so step ``s``
reads the original K/V block of ring rank ``(j - s) mod R`` instead of forwarding blocks hop by hop.
On the library path that read is an all-gather of K/V; dK/dV are accumulated in fp32 per source
block and reduce-scattered once (the reference's dependency passes fp32 dK/dV around the ring R
times).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch.autograd import Function

from ..comm import torch_backend as C
from ..ops import functional as F
from ..ops import native, torch_ref


# ----------------------------------------------------------------------------- Ulysses all-to-all


def _seq_to_head(x: torch.Tensor, group) -> torch.Tensor:
    """[t, U*h, hd] (local tokens; heads grouped by destination rank) -> [U*t, h, hd]."""
    U = C.group_size(group)
    if U == 1:
        return x
    t, H, hd = x.shape
    send = x.view(t, U, H // U, hd).permute(1, 0, 2, 3).contiguous()      # [U, t, h, hd]
    recv = C.all_to_all_chunks(send, group)                                # recv[u] = tokens of rank u
    return recv.view(U * t, H // U, hd)


def _head_to_seq(x: torch.Tensor, group) -> torch.Tensor:
    """[U*t, h, hd] -> [t, U*h, hd]; inverse of ``_seq_to_head``."""
    U = C.group_size(group)
    if U == 1:
        return x
    T, h, hd = x.shape
    t = T // U
    send = x.reshape(U, t, h, hd).contiguous()                             # send[u] = tokens of rank u
    recv = C.all_to_all_chunks(send, group)                                # recv[u] = head group u
    return recv.permute(1, 0, 2, 3).reshape(t, U * h, hd)


class _SeqToHead(Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _seq_to_head(x, group)

    @staticmethod
    def backward(ctx, dy):
        return _head_to_seq(dy.contiguous(), ctx.group), None


class _HeadToSeq(Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _head_to_seq(x, group)

    @staticmethod
    def backward(ctx, dy):
        return _seq_to_head(dy.contiguous(), ctx.group), None


def seq_to_head(x: torch.Tensor, group) -> torch.Tensor:
    """Scatter heads / gather sequence over ``group`` (differentiable)."""
    if C.group_size(group) == 1:
        return x
    return _SeqToHead.apply(x, group)


def head_to_seq(x: torch.Tensor, group) -> torch.Tensor:
    """Scatter sequence / gather heads over ``group`` (differentiable)."""
    if C.group_size(group) == 1:
        return x
    return _HeadToSeq.apply(x, group)


# ----------------------------------------------------------------------------- zigzag ring attention


def _merge_(out: torch.Tensor, lse: torch.Tensor, o: torch.Tensor, l: torch.Tensor, row0: int) -> None:
    """Fold a partial result (o [t,H,hd], l [H,t]) into rows ``row0:`` of the fp32 running (out, lse)."""
    sl = slice(row0, row0 + o.shape[0])
    lse_old = lse[:, sl]
    lse_new = torch.logaddexp(lse_old, l)
    wa = torch.exp(lse_old - lse_new).transpose(0, 1).unsqueeze(-1)
    wb = torch.exp(l - lse_new).transpose(0, 1).unsqueeze(-1)
    out[sl] = out[sl] * wa + o.float() * wb
    lse[:, sl] = lse_new


def ring_attn_fwd(q, k, v, group, scale):
    """Zigzag ring forward -> (out [Tb,H,hd] in q.dtype, lse [H,Tb] fp32)."""
    R, j = C.group_size(group), C.group_rank(group)
    if R == 1:
        return F.attn_block_fwd(q, k, v, True, scale)
    Tb = q.shape[0]
    half = Tb // 2
    kv_all = C.all_gather_rows(torch.stack([k, v]).unsqueeze(0), group)     # [R, 2, Tb, Hkv, hd]
    o0, lse = F.attn_block_fwd(q, k, v, True, scale)
    out = o0.float()
    lse = lse.clone()
    for s in range(1, R):
        src = (j - s) % R
        ks, vs = kv_all[src, 0], kv_all[src, 1]
        if src < j:
            # the source's early chunk precedes both of ours; its late chunk follows both
            o, l = F.attn_block_fwd(q, ks[:half], vs[:half], False, scale)
            _merge_(out, lse, o, l, 0)
        else:
            # only our late chunk sees the source, and it sees all of it
            o, l = F.attn_block_fwd(q[half:], ks, vs, False, scale)
            _merge_(out, lse, o, l, half)
    return out.to(q.dtype), lse


def ring_attn_bwd(do, q, k, v, o, lse, group, scale):
    """Zigzag ring backward -> (dq, dk, dv); dk/dv already summed over the ring for OUR block."""
    R, j = C.group_size(group), C.group_rank(group)
    if R == 1:
        return F.attn_block_bwd(do, q, k, v, o, lse, True, scale)
    Tb = q.shape[0]
    half = Tb // 2
    kv_all = C.all_gather_rows(torch.stack([k, v]).unsqueeze(0), group)
    dkv = torch.zeros(kv_all.shape, dtype=torch.float32, device=q.device)
    dq, dk0, dv0 = F.attn_block_bwd(do, q, k, v, o, lse, True, scale)
    dq = dq.float()
    dkv[j, 0] += dk0
    dkv[j, 1] += dv0
    lse_hi = lse[:, half:].contiguous()
    for s in range(1, R):
        src = (j - s) % R
        ks, vs = kv_all[src, 0], kv_all[src, 1]
        if src < j:
            dqs, dks, dvs = F.attn_block_bwd(do, q, ks[:half], vs[:half], o, lse, False, scale)
            dq += dqs
            dkv[src, 0, :half] += dks
            dkv[src, 1, :half] += dvs
        else:
            dqs, dks, dvs = F.attn_block_bwd(do[half:], q[half:], ks, vs, o[half:], lse_hi, False, scale)
            dq[half:] += dqs
            dkv[src, 0] += dks
            dkv[src, 1] += dvs
    mine = C.reduce_scatter_rows(dkv, group)[0]                               # [2, Tb, Hkv, hd]
    return dq, mine[0], mine[1]


class _ZigzagRingAttention(Function):
    @staticmethod
    def forward(ctx, q, k, v, group, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out, lse = ring_attn_fwd(q, k, v, group, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.group, ctx.scale = group, scale
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = ring_attn_bwd(do.contiguous(), q, k, v, o, lse, ctx.group, ctx.scale)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None


def zigzag_ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None,
                          scale: Optional[float] = None) -> torch.Tensor:
    """Causal attention over a sequence whose ring blocks are zigzag-sharded over ``group``.

    q [Tb, H, hd], k/v [Tb, Hkv, hd] hold this ring rank's block (chunks j and 2R-1-j of the global
    sequence, concatenated).  Same contract as the reference's dependency
    ``zigzag_ring_flash_attn_func(q, k, v, causal=True)`` without the batch dim."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _ZigzagRingAttention.apply(q, k, v, group, scale)


# ----------------------------------------------------------------------------- packed RoPE + attention


def _rope_inplace_(x3: torch.Tensor, n_rot: int, cos, sin, inverse: bool) -> None:
    """Rotate heads [0, n_rot) of the packed tensor x3 [T, heads, hd] in place."""
    if native.use_native(x3):
        native.lib().rope_inplace_(x3, n_rot, cos, sin, inverse)
    else:
        x3[:, :n_rot] = torch_ref.rope_apply(x3[:, :n_rot], cos, sin, inverse)


_rope_grouped = F.rope_grouped_


class _PackedRopeAttention(Function):
    @staticmethod
    def forward(ctx, qkv2d, cos, sin, hq, hkv, ring_group, scale, pre_rotated=False):
        Tb = qkv2d.shape[0]
        hd = qkv2d.shape[1] // (hq + 2 * hkv)
        # The producer of qkv2d (a GEMM) does not keep its output for backward, so rotating it in
        # place is invisible to autograd; the rotated tensor is what this op saves.
        qkv = qkv2d.detach().view(Tb, hq + 2 * hkv, hd)
        if not pre_rotated:
            _rope_inplace_(qkv, hq + hkv, cos, sin, False)
        q, k, v = qkv[:, :hq], qkv[:, hq:hq + hkv], qkv[:, hq + hkv:]
        if C.group_size(ring_group) > 1:
            from ..ops import fused_comm
            if fused_comm.ring_enabled(qkv, ring_group):
                o, lse = fused_comm.ring_attn_fwd(q, k, v, ring_group, scale)
            else:
                o, lse = ring_attn_fwd(q.contiguous(), k.contiguous(), v.contiguous(), ring_group, scale)
        else:
            o, lse = F.attn_block_fwd(q, k, v, True, scale)
        ctx.save_for_backward(qkv, cos, sin, o, lse)
        ctx.hq, ctx.hkv, ctx.ring_group, ctx.scale = hq, hkv, ring_group, scale
        return o.view(Tb, hq * hd)

    @staticmethod
    def backward(ctx, do2d):
        qkv, cos, sin, o, lse = ctx.saved_tensors
        hq, hkv, ring_group, scale = ctx.hq, ctx.hkv, ctx.ring_group, ctx.scale
        Tb, _, hd = qkv.shape
        do = do2d.contiguous().view(Tb, hq, hd)
        q, k, v = qkv[:, :hq], qkv[:, hq:hq + hkv], qkv[:, hq + hkv:]
        dqkv = torch.empty_like(qkv)
        if C.group_size(ring_group) > 1:
            from ..ops import fused_comm
            if fused_comm.ring_enabled(qkv, ring_group):
                fused_comm.ring_attn_bwd(do, q, k, v, o, lse, ring_group, scale, dqkv=dqkv)
            else:
                dq, dk, dv = ring_attn_bwd(do, q.contiguous(), k.contiguous(), v.contiguous(), o, lse,
                                           ring_group, scale)
                dqkv[:, :hq] = dq
                dqkv[:, hq:hq + hkv] = dk
                dqkv[:, hq + hkv:] = dv
        elif native.use_native(qkv) and native.has_native_attention_bwd() and hd == 128:
            # the kernel writes dq/dk/dv straight into the packed gradient
            native.lib().attn_bwd(do, q, k, v, o, lse, True, scale,
                                  dqkv[:, :hq], dqkv[:, hq:hq + hkv], dqkv[:, hq + hkv:])
        else:
            dq, dk, dv = F.attn_block_bwd(do, q, k, v, o, lse, True, scale)
            dqkv[:, :hq] = dq
            dqkv[:, hq:hq + hkv] = dk
            dqkv[:, hq + hkv:] = dv
        # also when the projection rotated q and k itself (pre_rotated): what goes back to it is the gradient of
        # its product before the rotation
        _rope_inplace_(dqkv, hq + hkv, cos, sin, True)
        return dqkv.view(Tb, -1), None, None, None, None, None, None, None


def packed_rope_attention(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, hq: int, hkv: int,
                          ring_group=None, scale: Optional[float] = None, pre_rotated: bool = False) -> torch.Tensor:
    """qkv [Tb, (hq + 2 hkv) * hd] laid out [q heads | k heads | v heads] per token, *consumed*
    (rotated in place).  cos/sin [Tb, hd/2] for the tokens' global positions.  Returns the
    attention output [Tb, hq * hd] of causal attention over the whole sequence (across
    ``ring_group`` when given).  ``pre_rotated``: the projection that produced ``qkv`` already rotated q and k in its
    epilogue (``parallel.linear.ag_linear(..., rope=...)``); the forward rotation is skipped, the backward one is not."""
    hd = qkv.shape[1] // (hq + 2 * hkv)
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    return _PackedRopeAttention.apply(qkv, cos, sin, hq, hkv, ring_group, scale, pre_rotated)
