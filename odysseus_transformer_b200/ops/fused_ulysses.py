"""DeepSpeed-Ulysses attention block whose four all-to-alls live inside the producing kernels (sm_100a).

The reference runs the sequence<->head exchange as separate ``all_to_all_single`` calls with
transposes and ``contiguous()`` copies around them (``yunchang`` ``SeqAllToAll4D``, called at reference
``decoder/ulysses.py:40-47``; four exchanges forward, four backward).  Here every exchange is the
epilogue of the kernel that produces the data, storing straight into the destination rank's receive
buffer over NVLink:

=========================  ==========================================================================
exchange                   producer kernel
=========================  ==========================================================================
forward  q,k,v seq->head   QKV projection GEMM (ZeRO-3 weight gather fused as well): ``gemm_comm``
                           with the all-to-all epilogue - column group ``u`` of a tile goes to rank ``u``,
                           q and k rotated (RoPE) on the way out of the accumulator
forward  o head->seq       attention forward: each CTA's output tile is stored to the rank owning those rows
backward do seq->head      output-projection dgrad GEMM with the all-to-all epilogue
backward dq,dk,dv          attention backward kernels store each gradient tile to the rank owning the rows
=========================  ==========================================================================

Receivers wait (bounded, one small kernel) on per-source arrival words before the consumer kernel
is launched, and tell the senders through ``consumed`` epoch words when a buffer may be overwritten.
One autograd function covers the whole block, so no gradient ever exists in a layout autograd would
have to understand.  Requirements: bf16, head_dim 128, local tokens a multiple of 128, symmetric heaps
for the weight group and the exchange group; otherwise ``available`` is False and the module runs the
torch.distributed composition.

Inner x ring hybrid (ring degree > 1, the layout the reference README only claims, reference
``README.md:14``): the attention core is the zigzag ring attention of ``ops.fused_comm`` (K/V pushed by
comm warps inside the attention kernels).  Its output is merged over ring steps by a separate kernel,
so the two exchanges that follow attention (o forward, dq/dk/dv backward) cannot ride an attention
epilogue; they run as one NCCL all-to-all each, while the two exchanges that follow a GEMM (q/k/v
forward, dO backward) stay in the GEMM epilogues.
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import fused_comm as FC
from . import native


def available(mod, x: torch.Tensor) -> bool:
    pc = mod.pctx
    if pc.inner_size < 2 or mod.head_dim != 128 or x.shape[0] % 128:
        return False
    if not (FC.enabled(x, pc.inner_group) and FC.enabled(x, pc.world_group)):
        return False
    if pc.ring_size > 1 and not FC.enabled(x, pc.ring_group):
        return False
    return native.has_native_attention() and native.has_native_attention_bwd()


def _need(v, what: str):
    if v is None:
        raise RuntimeError(f"fused Ulysses block: symmetric heap exhausted while allocating {what}; "
                           "give comm.symm.setup_fused_comm a larger data_bytes")
    return v


def _gather_w(heap, sched, idx, step, w, other, layout, scatter=None, rope=None, residual=None):
    """ZeRO-3 weight gather fused with its GEMM (operand B), riding the prefetch chain of ``sched``."""
    slot, nxt_w, nxt = FC._chain(sched, heap, idx, step, w)
    y, _, nslot = FC._gather_gemm(heap, w, 2, other, layout, slot=slot, prefetch=nxt_w, scatter=scatter, rope=rope,
                                  residual=residual)
    if nslot is not None:
        sched._fused_prefetched[nxt] = nslot
    return _need(y, "a weight gather buffer")


class _FusedUlyssesAttention(Function):
    @staticmethod
    def forward(ctx, x, wqkv, wo, cos, sin, mod, residual=None):
        from . import functional as F
        lib = native.lib()
        pc = mod.pctx
        heap_w, heap_a = FC.heap_for(pc.world_group), FC.heap_for(pc.inner_group)
        U, r = heap_a.n, heap_a.rank
        t, hq, hkv = x.shape[0], mod.hq, mod.hkv
        nh = hq + 2 * hkv
        G, Tb = nh * 128, U * t
        everyone = (1 << U) - 1
        sched, iq, io = mod.qkv_proj.sched, mod.qkv_proj.idx, mod.o_proj.idx
        x = x.contiguous()
        flag_dev = heap_a.local

        # 1. QKV projection; the epilogue scatters head group u to rank u (rows r*t.. of its [Tb, G] buffer)
        s_qkv = _need(heap_a.a2a_slot(Tb, G, "qkv"), "the q/k/v receive buffer")
        desc = s_qkv.gemm_desc(G, r * t, 0, FC._n_cta(heap_w, t, U * G))
        in_gemm = F.epilogue_fusion("rope")
        # q and k are rotated in the GEMM epilogue, at this rank's own token positions, before they cross the link
        rope = F.RopeEpilogue(cos[r * t:(r + 1) * t], sin[r * t:(r + 1) * t], (hq + hkv) * 128, G) if in_gemm else None
        _gather_w(heap_w, sched, iq, +1, wqkv.detach(), x, 0, scatter=desc, rope=rope)
        lib.wait_flags(flag_dev, s_qkv.arrived_local(), everyone, s_qkv.arrived_total)
        # out of the receive buffer in one pass (rotating on the way when the epilogue did not); the copy is kept for
        # backward and the buffer is free again at once
        qkv3 = torch.empty(Tb, nh, 128, dtype=x.dtype, device=x.device)
        if in_gemm:
            qkv3.copy_(s_qkv.local().view(Tb, nh, 128))
        else:
            F.rope_grouped_(s_qkv.local().view(Tb, nh, 128), qkv3, hq + hkv, nh, cos, sin, False)
        qkv = qkv3.view(Tb, G)
        lib.signal_flags(flag_dev, s_qkv.consumed_ptrs(), everyone, r, s_qkv.uses)
        q, k, v = qkv3[:, :hq], qkv3[:, hq:hq + hkv], qkv3[:, hq + hkv:]

        scale = mod.head_dim ** -0.5
        if pc.ring_size > 1:
            # 2'. hybrid: zigzag ring attention over the ring group, then the head -> sequence exchange as one all-to-all
            from ..parallel.attention import _head_to_seq
            o, lse = FC.ring_attn_fwd(q, k, v, pc.ring_group, scale)
            o_seq = _head_to_seq(o, pc.inner_group).reshape(t, U * hq * 128)
        else:
            # 2. attention; each output tile also goes to the rank that owns its rows (columns of head group r there)
            s_o = _need(heap_a.a2a_slot(t, U * hq * 128, "o"), "the attention-output receive buffer")
            e_o = s_o.begin_epoch()
            lib.wait_flags(flag_dev, s_o.consumed_local(), everyone, e_o - 1)
            dests = [s_o.on_peer(p).view(t, U, hq, 128)[:, r] for p in range(U)]
            o, lse = lib.attn_fwd_split(q, k, v, True, scale, dests)
            lib.signal_flags(flag_dev, s_o.arrived_ptrs(), everyone, r, e_o)
            lib.wait_flags(flag_dev, s_o.arrived_local(), everyone, e_o)
            o_seq = s_o.local().clone()                     # [t, H * 128], kept for the o_proj wgrad
            lib.signal_flags(flag_dev, s_o.consumed_ptrs(), everyone, r, e_o)

        # 3. output projection (ZeRO-3 weight gather fused)
        if residual is not None and residual.stride(-1) != 1:
            residual = residual.contiguous()
        y = _gather_w(heap_w, sched, io, +1, wo.detach(), o_seq, 0, residual=residual)
        ctx.save_for_backward(x, wqkv, wo, cos, sin, qkv, o, lse, o_seq)
        ctx.mod = mod
        FC.stats["ulysses"] = FC.stats.get("ulysses", 0) + 1
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..parallel.attention import _rope_grouped, _rope_inplace_
        x, wqkv, wo, cos, sin, qkv, o, lse, o_seq = ctx.saved_tensors
        mod = ctx.mod
        lib = native.lib()
        pc = mod.pctx
        heap_w, heap_a = FC.heap_for(pc.world_group), FC.heap_for(pc.inner_group)
        U, r = heap_a.n, heap_a.rank
        t, hq, hkv = x.shape[0], mod.hq, mod.hkv
        nh = hq + 2 * hkv
        G, Tb = nh * 128, U * t
        everyone = (1 << U) - 1
        sched, iq, io = mod.qkv_proj.sched, mod.qkv_proj.idx, mod.o_proj.idx
        flag_dev = heap_a.local
        dy = dy.contiguous()

        # 1. o_proj dgrad; the epilogue scatters the columns of head group u to rank u: dO arrives as [Tb, hq * 128]
        s_do = _need(heap_a.a2a_slot(Tb, hq * 128, "do"), "the dO receive buffer")
        desc = s_do.gemm_desc(hq * 128, r * t, 0, FC._n_cta(heap_w, t, U * hq * 128))
        _gather_w(heap_w, sched, io, -1, wo.detach(), dy, 1, scatter=desc)
        g_wo = FC.zero3_wgrad(heap_w, pc.world_group, wo, dy, o_seq)
        lib.wait_flags(flag_dev, s_do.arrived_local(), everyone, s_do.arrived_total)
        do = s_do.local().view(Tb, hq, 128)

        qkv3 = qkv.view(Tb, nh, 128)
        q, k, v = qkv3[:, :hq], qkv3[:, hq:hq + hkv], qkv3[:, hq + hkv:]
        scale = mod.head_dim ** -0.5
        hybrid = pc.ring_size > 1
        if hybrid:
            # 2'. hybrid: ring attention backward into a local packed gradient, inverse rotation at the block's positions,
            # then the head -> sequence exchange of the packed gradient as one all-to-all
            from ..parallel.attention import _head_to_seq
            dq3 = torch.empty_like(qkv3)
            FC.ring_attn_bwd(do, q, k, v, o, lse, pc.ring_group, scale, dqkv=dq3)
            lib.signal_flags(flag_dev, s_do.consumed_ptrs(), everyone, r, s_do.uses)
            _rope_inplace_(dq3, hq + hkv, cos, sin, True)
            dqkv = _head_to_seq(dq3, pc.inner_group).reshape(t, U * G)
        else:
            # 2. attention backward; gradient tiles go to the rank owning the rows, landing packed as [t, U * G]
            s_dqkv = _need(heap_a.a2a_slot(t, U * G, "dqkv"), "the dq/dk/dv receive buffer")
            e = s_dqkv.begin_epoch()
            lib.wait_flags(flag_dev, s_dqkv.consumed_local(), everyone, e - 1)
            there = [s_dqkv.on_peer(p).view(t, U, nh, 128)[:, r] for p in range(U)]
            lib.attn_bwd_split(do, q, k, v, o, lse, True, scale, [d[:, :hq] for d in there],
                               [d[:, hq:hq + hkv] for d in there], [d[:, hq + hkv:] for d in there])
            lib.signal_flags(flag_dev, s_do.consumed_ptrs(), everyone, r, s_do.uses)
            lib.signal_flags(flag_dev, s_dqkv.arrived_ptrs(), everyone, r, e)
            lib.wait_flags(flag_dev, s_dqkv.arrived_local(), everyone, e)
            dqkv = s_dqkv.local()
            # inverse rotation of the dq / dk heads of every head group, at this rank's own token positions
            cos_l, sin_l = cos[r * t:(r + 1) * t], sin[r * t:(r + 1) * t]
            by_group = dqkv.view(t, U * nh, 128)
            _rope_grouped(by_group, by_group, hq + hkv, nh, cos_l, sin_l, True)

        # 3. QKV projection backward, reading the receive buffer in place
        dx = _gather_w(heap_w, sched, iq, -1, wqkv.detach(), dqkv, 1)
        g_wqkv = FC.zero3_wgrad(heap_w, pc.world_group, wqkv, dqkv, x)
        if not hybrid:
            lib.signal_flags(flag_dev, s_dqkv.consumed_ptrs(), everyone, r, e)
        return dx, g_wqkv, g_wo, None, None, None, (dy if ctx.needs_input_grad[6] else None)


def attention_block(mod, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, residual=None) -> torch.Tensor:
    """``SequenceParallelAttention.forward`` on the fused path: x [t, d] local tokens -> [t, d] (+ residual, added in
    the output projection's epilogue)."""
    return _FusedUlyssesAttention.apply(x, mod.qkv_proj.weight, mod.o_proj.weight, cos, sin, mod, residual)
