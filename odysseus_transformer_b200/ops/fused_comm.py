"""Single-kernel compute+collective paths over NVLink peer memory (sm_100a only).

``enabled(x, group)`` says whether the fused kernels serve this call: CUDA bf16 tensors, a backend other
than ``library``, a multi-rank group and a symmetric heap registered for that group
(``comm.symm.setup_fused_comm``).  Otherwise callers run the torch.distributed + GEMM composition in
``parallel.linear``.  Each autograd function below replaces a collective + GEMM pair of the reference by
ONE launch of ``csrc/gemm_comm.cu``:

=====================  ===============================  =========================================
op                     forward                          backward
=====================  ===============================  =========================================
``ag_linear``          all-gather(x) -> GEMM            dgrad GEMM -> reduce-scatter ;
(column parallel)      (reference linear_tpsp.py:159-173)  all-gather(x) -> wgrad GEMM (:205-298)
``linear_rs``          GEMM -> reduce-scatter           all-gather(dy) -> dgrad GEMM ; wgrad GEMM on
(row parallel)         (reference linear_tpsp.py:588-591)  the gathered dy (:97, autograd of F.linear)
``zero3_linear``       all-gather(W) -> GEMM            all-gather(W) -> dgrad GEMM ;
                       (reference linear_zero3.py:35-44)   wgrad GEMM -> reduce-scatter (:62-84)
=====================  ===============================  =========================================

A shape the kernels do not take (shard rows not a multiple of 64, heap exhausted) falls back, op by op,
to the unfused function.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch.autograd import Function

from . import native

_heaps = {}   # id(group) -> comm.symm.SymmetricHeap
stats = {"gather": 0, "scatter": 0, "fallback": 0}   # fused launches / per-op fallbacks since import


def register_heap(group, heap) -> None:
    _heaps[id(group)] = heap


def heap_for(group):
    return _heaps.get(id(group))


def clear_heaps() -> None:
    _heaps.clear()


def enabled(x, group) -> bool:
    if group is None or not x.is_cuda or x.dtype != torch.bfloat16 or native.get_backend() == "library":
        return False
    return id(group) in _heaps and native.available()


def ring_enabled(x, group) -> bool:
    """Ring attention whose attention kernels carry the K/V exchange (``ring_attn_fwd`` below): packed
    ``[Tb, heads, 128]`` input with Tb a multiple of 128 and a heap for the ring group."""
    return (enabled(x, group) and x.dim() == 3 and x.shape[-1] == 128 and x.shape[0] % 128 == 0
            and native.has_native_attention() and native.has_native_attention_bwd())


def _lib():
    return native.lib()


def _n_cta(heap, M: int, N: int) -> int:
    return min(((M + 127) // 128) * ((N + 255) // 256), heap.sm_count)


def _push_only(heap, shard: torch.Tensor):
    """Deliver ``shard`` into every rank's gathered buffer with a push-only launch; returns the slot."""
    shard = shard if shard.stride(-1) == 1 else shard.contiguous()
    slot = heap.gather_slot(shard.shape[0], shard.shape[1])
    if slot is None:
        return None
    _lib().push_shard(slot.push_desc(shard, heap.sm_count))
    stats["push_only"] = stats.get("push_only", 0) + 1
    return slot


def _gather_gemm(heap, shard: torch.Tensor, which: int, other: torch.Tensor, layout: int,
                 out: Optional[torch.Tensor] = None, slot=None, prefetch: Optional[torch.Tensor] = None, scatter=None,
                 rope=None, residual: Optional[torch.Tensor] = None):
    """GEMM whose operand ``which`` (1 = A, 2 = B) is the all-gather of ``shard``.

    ``slot``: the gathered buffer when an earlier launch already delivered ``shard`` (prefetch), else the
    comm warps of THIS launch deliver it.  ``prefetch``: another shard for this launch's comm warps to
    deliver when they have nothing else to do (only possible when ``slot`` was given).
    ``scatter``: an all-to-all description (``comm.symm.A2ASlot.gemm_desc``) for the epilogue; the result
    is then the local receive buffer, complete only after a wait on the slot's arrival words.
    ``rope`` (``ops.functional.RopeEpilogue``; layout 0) / ``residual`` ([M, N]; not with ``scatter``): applied to
    the product in the epilogue.  A ``rope`` the kernel cannot take (head_dim other than 128) makes the call unsupported.
    Returns (result, gathered view, slot holding the prefetched shard or None); result None = unsupported."""
    shard = shard if shard.stride(-1) == 1 else shard.contiguous()
    pushed = slot is not None
    if rope is not None and not rope.in_kernel((shard.shape[0] * heap.n) if which == 2 else other.shape[0]):
        if slot is None:
            stats["fallback"] += 1
            return None, None, None
        raise RuntimeError("fused GEMM: the rotary epilogue needs head_dim 128")
    if slot is None:
        slot = heap.gather_slot(shard.shape[0], shard.shape[1])
        if slot is None:
            stats["fallback"] += 1
            return None, None, None
    stats["gather"] += 1
    g = slot.view()
    a, b = (g, other) if which == 1 else (other, g)
    M = a.shape[1] if layout == 2 else a.shape[0]
    N = b.shape[0] if layout == 0 else b.shape[1]
    n_cta = _n_cta(heap, M, N)
    push, next_slot = None, None
    if not pushed:
        push = slot.push_desc(shard, n_cta)
    elif prefetch is not None:
        prefetch = prefetch if prefetch.stride(-1) == 1 else prefetch.contiguous()
        next_slot = heap.gather_slot(prefetch.shape[0], prefetch.shape[1])
        if next_slot is not None:
            push = next_slot.push_desc(prefetch, n_cta)
            stats["prefetch"] = stats.get("prefetch", 0) + 1
    if rope is None and residual is None:
        y = _lib().gemm_comm(a, b, out, layout, slot.consume_desc(which, n_cta), push, scatter)
    else:
        y = _lib().gemm_comm(a, b, out, layout, slot.consume_desc(which, n_cta), push, scatter,
                             tuple(rope) if rope is not None else None, residual)
    return y, g, next_slot


def _scatter_gemm(heap, a: torch.Tensor, b: torch.Tensor, layout: int, M: int, N: int,
                  out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None):
    """GEMM whose [M, N] result is reduce-scattered on rows; returns this rank's [M/n, N] or None.
    ``residual`` [M/n, N] starts the sum of this rank's rows."""
    if M % heap.n:
        stats["fallback"] += 1
        return None
    chunk = M // heap.n
    slot = heap.scatter_slot(chunk, N)
    if slot is None:
        stats["fallback"] += 1
        return None
    stats["scatter"] += 1
    if out is None:
        out = torch.empty(chunk, N, dtype=a.dtype, device=a.device)
    if residual is None:
        _lib().gemm_comm(a, b, None, layout, None, None, slot.describe(out))
    else:
        residual = residual if residual.stride(-1) == 1 else residual.contiguous()
        _lib().gemm_comm(a, b, None, layout, None, None, slot.describe(out), None, residual)
    return out


# ----------------------------------------------------------------------------- column parallel


class _FusedAGLinear(Function):
    @staticmethod
    def forward(ctx, x, w, group, rope=None):
        from ..ops import functional as F
        heap = heap_for(group)
        ctx.group = group
        ctx.save_for_backward(x, w)
        y, _, _ = _gather_gemm(heap, x, 1, w, 0, rope=rope)
        if y is None:
            from ..comm import torch_backend as C
            y = F.gemm_nt(C.all_gather_rows(x, group), w, rope=rope)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..comm import torch_backend as C
        from ..ops import functional as F
        x, w = ctx.saved_tensors
        heap = heap_for(ctx.group)
        dy = dy.contiguous()
        # dX = reduce-scatter(dY @ W)
        dx = _scatter_gemm(heap, dy, w, 1, dy.shape[0], w.shape[1])
        if dx is None:
            dx = C.reduce_scatter_rows(F.gemm_nn(dy, w), ctx.group)
        # dW = dY^T @ all-gather(x): the gathered x streams in along K
        mg = getattr(w, "main_grad", None)
        fresh = mg is not None and not getattr(w, "_grad_written", False)
        dw, _, _ = _gather_gemm(heap, x, 2, dy, 2, out=mg if fresh else None)
        if dw is None:
            return dx, F.store_weight_grad(w, dy, C.all_gather_rows(x, ctx.group)), None, None
        if fresh:
            w._grad_written = True
            return dx, None, None, None
        return dx, F.deliver_grad(w, dw), None, None


def ag_linear(x: torch.Tensor, w: torch.Tensor, group, rope=None) -> torch.Tensor:
    return _FusedAGLinear.apply(x, w, group, rope)


# ----------------------------------------------------------------------------- row parallel


class _FusedLinearRS(Function):
    @staticmethod
    def forward(ctx, x, w, group, residual=None):
        from ..comm import torch_backend as C
        from ..ops import functional as F
        heap = heap_for(group)
        ctx.group = group
        ctx.save_for_backward(x, w)
        x = x if x.stride(-1) == 1 else x.contiguous()
        y = _scatter_gemm(heap, x, w, 0, x.shape[0], w.shape[0], residual=residual)
        if y is None:
            y = C.reduce_scatter_rows(F.gemm_nt(x, w), group)
            if residual is not None:
                y.add_(residual)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..comm import torch_backend as C
        from ..ops import functional as F
        x, w = ctx.saved_tensors
        heap = heap_for(ctx.group)
        dy = dy.contiguous()
        # dX = all-gather(dY) @ W ; the gathered dY stays in the slot for the wgrad GEMM that follows
        dx, dy_full, _ = _gather_gemm(heap, dy, 1, w, 1)
        if dx is None:
            dy_full = C.all_gather_rows(dy, ctx.group)
            dx = F.gemm_nn(dy_full, w)
        dw = F.store_weight_grad(w, dy_full, x)
        return dx, dw, None, (dy if ctx.needs_input_grad[3] else None)


def linear_rs(x: torch.Tensor, w: torch.Tensor, group, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _FusedLinearRS.apply(x, w, group, residual)


# ----------------------------------------------------------------------------- ZeRO-3


def _chain(sched, heap, idx: int, step: int, w: torch.Tensor):
    """Prefetch bookkeeping of a ZeRO-3 linear: (slot already holding all-gather(w) or None, next weight to
    prefetch or None, its index).  Weights register in forward order in ``sched``; forward walks +1, backward
    -1.  The first linear of a pass has no earlier GEMM to ride on and starts the chain with a push-only launch."""
    if sched is None or not getattr(sched, "enabled", True):
        return None, None, None
    pre = sched.__dict__.setdefault("_fused_prefetched", {})
    slot = pre.pop(idx, None)
    nxt = idx + step
    nxt_w = None
    if 0 <= nxt < len(sched.weights) and sched.groups[nxt] is sched.groups[idx] and nxt not in pre:
        cand = sched.weights[nxt].detach()
        if cand.is_cuda and cand.dtype == torch.bfloat16 and cand.shape[0] % 64 == 0 and cand.shape[1] % 64 == 0:
            nxt_w = cand
    if slot is None and nxt_w is not None:
        slot = _push_only(heap, w)          # may be None (unsupported shape): then this op pushes in-kernel
    return slot, nxt_w, nxt


class _FusedZero3Linear(Function):
    @staticmethod
    def forward(ctx, x, w, group, sched, idx, rope=None, residual=None):
        from ..comm import torch_backend as C
        from ..ops import functional as F
        heap = heap_for(group)
        ctx.group, ctx.sched, ctx.idx = group, sched, idx
        ctx.save_for_backward(x, w)
        x = x if x.stride(-1) == 1 else x.contiguous()
        if residual is not None and residual.stride(-1) != 1:
            residual = residual.contiguous()
        slot, nxt_w, nxt = _chain(sched, heap, idx, +1, w.detach())
        if rope is not None and not rope.in_kernel(w.shape[0] * heap.n):
            # head_dim other than 128: the rotation is a pass of its own after the fused GEMM
            y, full, nslot = _gather_gemm(heap, w.detach(), 2, x, 0, slot=slot, prefetch=nxt_w, residual=residual)
            if y is not None:
                F.apply_rope_epilogue_(y, rope)
        else:
            y, full, nslot = _gather_gemm(heap, w.detach(), 2, x, 0, slot=slot, prefetch=nxt_w, rope=rope, residual=residual)
        if nslot is not None:
            sched._fused_prefetched[nxt] = nslot
        if y is None:
            full = C.all_gather_rows(w.detach(), group)
            y = F.gemm_nt(x, full, rope=rope, residual=residual)
        if sched is not None and sched.keep_gathered and any(ctx.needs_input_grad):
            # ZeRO-2 style (the reference's --use_zero2, train.py:137-141): the whole weight stays resident until
            # this layer's backward, which then needs no second gather.  The slot itself is recycled, so copy.
            sched._kept[idx] = full.clone()
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..comm import torch_backend as C
        from ..ops import functional as F
        x, w = ctx.saved_tensors
        group, sched, idx = ctx.group, ctx.sched, ctx.idx
        heap = heap_for(group)
        dy = dy.contiguous()
        kept = sched._kept.pop(idx, None) if (sched is not None and sched.keep_gathered) else None
        d_res = dy if ctx.needs_input_grad[6] else None
        if kept is not None:
            dx = F.gemm_nn(dy, kept) if ctx.needs_input_grad[0] else None
            return dx, zero3_wgrad(heap, group, w, dy, x), None, None, None, None, d_res
        slot, nxt_w, nxt = _chain(sched, heap, idx, -1, w.detach())
        dx = None
        if ctx.needs_input_grad[0] or slot is not None:
            dx, _, nslot = _gather_gemm(heap, w.detach(), 2, dy, 1, slot=slot, prefetch=nxt_w)   # W streams in along K
            if nslot is not None:
                sched._fused_prefetched[nxt] = nslot
            if dx is None:
                dx = F.gemm_nn(dy, C.all_gather_rows(w.detach(), group))
        return dx, zero3_wgrad(heap, group, w, dy, x), None, None, None, None, d_res


def zero3_wgrad(heap, group, w, dy, x):
    """Weight gradient of a ZeRO-3 linear: wgrad GEMM -> reduce-scatter in one kernel, written straight into
    ``w.main_grad`` when that is fresh.  Returns what autograd should receive for ``w``."""
    from ..comm import torch_backend as C
    from ..ops import functional as F
    mg = getattr(w, "main_grad", None)
    fresh = mg is not None and not getattr(w, "_grad_written", False)
    dw = _scatter_gemm(heap, dy, x, 2, heap.n * w.shape[0], w.shape[1], out=mg if fresh else None)
    if dw is None:
        dw = C.reduce_scatter_rows(F.gemm_tn(dy, x), group)
        return F.deliver_grad(w, dw)
    if fresh:
        w._grad_written = True
        return None
    return F.deliver_grad(w, dw)


def zero3_linear(x: torch.Tensor, w_shard: torch.Tensor, group, sched=None, idx: int = 0, rope=None,
                 residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _FusedZero3Linear.apply(x, w_shard, group, sched, idx, rope, residual)


# ----------------------------------------------------------------------------- zigzag ring attention


def _kv_shard(k: torch.Tensor, v: torch.Tensor) -> Optional[torch.Tensor]:
    """The rows ``[k heads | v heads]`` of the packed qkv tensor as one strided [Tb, 2 * hkv * 128] view."""
    Tb, hkv, hd = k.shape
    adjacent = (v.data_ptr() == k.data_ptr() + hkv * hd * k.element_size() and k.stride() == v.stride()
                and k.stride(1) == hd and k.stride(2) == 1 and k.stride(0) >= 2 * hkv * hd)
    if not adjacent:
        return None
    return torch.as_strided(k, (Tb, 2 * hkv * hd), (k.stride(0), 1))


def _ring_setup(q, k, v, group):
    heap = _heaps[id(group)]
    shard = _kv_shard(k, v)
    slot = heap.gather_slot(k.shape[0], 2 * k.shape[1] * k.shape[2], tag="ring") if shard is not None else None
    return heap, shard, slot


def ring_attn_fwd(q, k, v, group, scale):
    """Zigzag ring forward over peer memory -> (out [Tb, H, 128] bf16, lse [H, Tb] fp32).

    The reference's dependency passes K/V blocks hop by hop with batched isend/irecv between attention
    calls (``zigzag_ring_flash_attn_func``, called at reference ``decoder/ring.py:30-37``).  Here the
    attention kernel of ring step ``s`` carries comm warps that store this rank's K/V rows straight into
    the buffer of the rank ``s + 1`` places downstream - the rank whose step ``s + 1`` reads them - so
    every transfer is hidden behind one step of tensor-core work and crosses NVSwitch exactly once.  A
    one-thread kernel in front of step ``s`` waits (bounded) for that step's source to have arrived.  The
    R partial results are merged in one pass at the end."""
    from ..parallel import attention as PA
    heap, shard, slot = _ring_setup(q, k, v, group)
    if slot is None:
        stats["fallback"] += 1
        return PA.ring_attn_fwd(q.contiguous(), k.contiguous(), v.contiguous(), group, scale)
    lib = _lib()
    R, j = heap.n, heap.rank
    Tb, hq = q.shape[0], q.shape[1]
    half = Tb // 2
    # the push is spread over every CTA of the smaller step grid: a CTA's comm warps then finish with its tiles
    n_push = min(int(lib.attn_fwd_ctas(half, hq)), 4096)
    base = slot.push_desc(shard, n_push)
    gathered = slot.view().view(R, Tb, 2, k.shape[1], 128)

    def push(step):
        d = dict(base)
        d["dest_first"], d["dest_count"] = step + 1, 1
        return d

    o, l = lib.attn_fwd_push(q, k, v, True, scale, push(0))
    os_, ls_, begins = [o], [l], [0]
    for s in range(1, R):
        src = (j - s) % R
        lib.wait_shard(base, src)
        ks, vs = gathered[src, :, 0], gathered[src, :, 1]
        # zigzag: an earlier source's first chunk precedes both of ours; a later source is seen, whole, by our late chunk only
        args = (q, ks[:half], vs[:half]) if src < j else (q[half:], ks, vs)
        if s < R - 1:
            o, l = lib.attn_fwd_push(*args, False, scale, push(s))
        else:
            o, l = lib.attn_fwd(*args, False, scale)
        os_.append(o)
        ls_.append(l)
        begins.append(0 if src < j else half)
    lib.signal_free(base)
    stats["ring"] = stats.get("ring", 0) + 1
    out, lse = lib.attn_merge_parts(os_, ls_, begins, Tb)
    return out, lse


def ring_attn_bwd(do, q, k, v, o, lse, group, scale, dqkv=None):
    """Zigzag ring backward.  Returns (dq, dk, dv), or fills the packed gradient ``dqkv [Tb, hq + 2 hkv, 128]``
    when it is given, with dk/dv summed over the ring for this rank's block.

    K/V are exchanged again (nothing gathered is kept between forward and backward): a push-only launch on
    a side stream delivers this rank's rows to every peer while the local causal block runs, and each later
    step waits for its source as in the forward.  The dK/dV that step ``s`` computes belong to the source
    rank: the backward kernel stores them straight into that rank's inbox over NVLink (its output tensors
    live in the peer's symmetric memory), an epoch word announces them, and every rank finally adds its R-1
    inboxes to its own dK/dV in one fp32 pass.  There is no reduce-scatter and no fp32 staging: the
    reference's dependency sends fp32 dK/dV around the ring R times."""
    from ..parallel import attention as PA
    heap, shard, slot = _ring_setup(q, k, v, group)
    Tb, hq, hkv = q.shape[0], q.shape[1], k.shape[1]
    inbox = heap.inbox_slot(Tb, 2 * hkv * 128) if slot is not None else None
    if inbox is None:
        stats["fallback"] += 1
        dq, dk, dv = PA.ring_attn_bwd(do, q.contiguous(), k.contiguous(), v.contiguous(), o, lse, group, scale)
        if dqkv is None:
            return dq, dk, dv
        dqkv[:, :hq], dqkv[:, hq:hq + hkv], dqkv[:, hq + hkv:] = dq, dk, dv
        return None
    lib = _lib()
    R, j = heap.n, heap.rank
    half = Tb // 2
    ret = dqkv is None
    if ret:
        dqkv = torch.empty((Tb, hq + 2 * hkv, 128), dtype=q.dtype, device=q.device)
    base = slot.push_desc(shard, heap.sm_count)
    base["dest_first"], base["dest_count"] = 1, R - 1
    epoch = inbox.begin()
    main = torch.cuda.current_stream()
    side = heap.side_stream()
    side.wait_stream(main)
    with torch.cuda.stream(side):
        lib.push_shard(base)
    gathered = slot.view().view(R, Tb, 2, hkv, 128)
    lib.attn_bwd(do, q, k, v, o, lse, True, scale, dqkv[:, :hq], dqkv[:, hq:hq + hkv], dqkv[:, hq + hkv:])
    do_hi, o_hi, lse_hi = do[half:], o[half:], lse[:, half:].contiguous()
    dq_parts, dq_begins = [], []
    for s in range(1, R):
        src = (j - s) % R
        lib.wait_shard(base, src)
        # the owner must have folded the previous contents of our inbox there into its gradient
        lib.wait_flags(heap.local, inbox.consumed_local(), 1 << src, epoch - 1)
        ks, vs = gathered[src, :, 0], gathered[src, :, 1]
        mine_there = inbox.on_peer(src)[j].view(Tb, 2, hkv, 128)
        if src < j:
            dqs = torch.empty((Tb, hq, 128), dtype=q.dtype, device=q.device)
            lib.attn_bwd(do, q, ks[:half], vs[:half], o, lse, False, scale, dqs, mine_there[:half, 0], mine_there[:half, 1])
            dq_begins.append(0)
        else:
            dqs = torch.empty((Tb - half, hq, 128), dtype=q.dtype, device=q.device)
            lib.attn_bwd(do_hi, q[half:], ks, vs, o_hi, lse_hi, False, scale, dqs, mine_there[:, 0], mine_there[:, 1])
            dq_begins.append(half)
        lib.signal_flags(heap.local, inbox.arrived_ptrs(), 1 << src, j, epoch)
        dq_parts.append(dqs.view(dqs.shape[0], hq * 128))
    lib.signal_free(base)
    main.wait_stream(side)
    others = ((1 << R) - 1) & ~(1 << j)
    lib.wait_flags(heap.local, inbox.arrived_local(), others, epoch)
    flat = dqkv.view(Tb, (hq + 2 * hkv) * 128)
    lib.sum_rows_(flat[:, :hq * 128], dq_parts, dq_begins)
    box = inbox.local()
    # a later ring rank sees only the first chunk of our keys; an earlier one sees all of them
    parts = [box[i, :half] if i > j else box[i] for i in range(R) if i != j]
    lib.sum_rows_(flat[:, hq * 128:], parts, [0] * len(parts))
    lib.signal_flags(heap.local, inbox.consumed_ptrs(), others, j, epoch)
    stats["ring"] = stats.get("ring", 0) + 1
    if ret:
        return dqkv[:, :hq], dqkv[:, hq:hq + hkv], dqkv[:, hq + hkv:]
    return None
