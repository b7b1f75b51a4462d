"""Communication-aware linear layers (the reference's L1 layer).

* ``ColumnParallelLinearAG`` - weight split on out-features; the input is the local sequence
  shard, all-gathered on the sequence dim inside the op (reference ``utils/linear_tpsp.py:405-500``,
  autograd function ``:125-303``).
* ``RowParallelLinearRS`` - weight split on in-features; the partial outputs are reduce-scattered on
  the sequence dim (reference ``utils/linear_tpsp.py:503-596``).
* ``LinearZeRO3`` - activations stay local; the *weight* is sharded on out-features, all-gathered
  before the forward and the backward GEMMs, and its gradient reduce-scattered with SUM
  (reference ``utils/linear_zero3.py:21-130``).
* ``all_gather_seq`` / ``reduce_scatter_seq`` - the differentiable collective pair
  (reference ``utils/allgather.py:4-10``, ``utils/linear_tpsp.py:84-111``).

Differences by design: the library path overlaps the same collectives the reference overlaps
(and the ZeRO-3 gathers/reduce-scatters it leaves exposed) using NCCL's async handles, not
``CUDA_DEVICE_MAX_CONNECTIONS=1`` ordering; weights are initialised or loaded from HF state-dict
tensors by the model loader (the reference leaves ``LinearZeRO3`` uninitialised,
``utils/linear_zero3.py:113-115``); on CUDA with the ``fused`` backend and a symmetric heap the
collective+GEMM pairs run as single kernels (``ops.fused_comm``).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn
from torch.autograd import Function

from ..comm import torch_backend as C
from ..ops import functional as F
from ..utils.buffers import get_global_memory_buffer

# async works whose results the optimizer needs (gradient reduce-scatters)
_PENDING: List[object] = []


def wait_pending_grad_comm() -> None:
    """Block the current stream until every in-flight gradient reduce-scatter has finished."""
    while _PENDING:
        w = _PENDING.pop()
        if w is not None:
            w.wait()


# ----------------------------------------------------------------------------- differentiable collectives


class _AllGatherSeq(Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return C.all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, dy):
        return C.reduce_scatter_rows(dy, ctx.group), None


class _ReduceScatterSeq(Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return C.reduce_scatter_rows(x, group)

    @staticmethod
    def backward(ctx, dy):
        return C.all_gather_rows(dy, ctx.group), None


def all_gather_seq(x: torch.Tensor, group) -> torch.Tensor:
    """[T/n, ...] -> [T, ...]; backward is a reduce-scatter (reference ``allgather_bsz1``)."""
    return _AllGatherSeq.apply(x, group)


def reduce_scatter_seq(x: torch.Tensor, group) -> torch.Tensor:
    """[T, ...] partial sums -> [T/n, ...]; backward is an all-gather."""
    return _ReduceScatterSeq.apply(x, group)


# ----------------------------------------------------------------------------- AG -> GEMM (column parallel)


class _AGLinear(Function):
    @staticmethod
    def forward(ctx, x, w, group):
        ctx.group = group
        ctx.save_for_backward(x, w)           # only the LOCAL shard of the input is kept
        n = C.group_size(group)
        if n == 1:
            return F.gemm_nt(x, w)
        buf = get_global_memory_buffer().get_tensor((n * x.shape[0], x.shape[1]), x.dtype, "mpu", x.device)
        total = C.all_gather_rows(x, group, out=buf)
        return F.gemm_nt(total, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        group = ctx.group
        n = C.group_size(group)
        dy = dy.contiguous()
        if n == 1:
            dx = F.gemm_nn(dy, w)
            return dx, F.store_weight_grad(w, dy, x), None
        # re-gather the input while the dgrad GEMM runs
        buf = get_global_memory_buffer().get_tensor((n * x.shape[0], x.shape[1]), x.dtype, "mpu", x.device)
        total, work = C.all_gather_rows(x, group, out=buf, async_op=True)
        dx_full = F.gemm_nn(dy, w)
        if work is not None:
            work.wait()
        # reduce-scatter dX while the wgrad GEMM runs
        dx, work = C.reduce_scatter_rows(dx_full, group, async_op=True)
        dw = F.store_weight_grad(w, dy, total)
        if work is not None:
            work.wait()
        return dx, dw, None


def ag_linear(x: torch.Tensor, w: torch.Tensor, group) -> torch.Tensor:
    """x [T/n, in] (sequence shard), w [out_local, in] -> [T, out_local]."""
    from ..ops import fused_comm
    if fused_comm.enabled(x, group):
        return fused_comm.ag_linear(x, w, group)
    return _AGLinear.apply(x, w, group)


# ----------------------------------------------------------------------------- GEMM -> RS (row parallel)


class _LinearRS(Function):
    @staticmethod
    def forward(ctx, x, w, group):
        ctx.group = group
        ctx.save_for_backward(x, w)
        y = F.gemm_nt(x, w)
        return C.reduce_scatter_rows(y, group)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        n = C.group_size(ctx.group)
        dy = dy.contiguous()
        if n > 1:
            buf = get_global_memory_buffer().get_tensor((n * dy.shape[0], dy.shape[1]), dy.dtype, "mpu", dy.device)
            dy = C.all_gather_rows(dy, ctx.group, out=buf)
        dx = F.gemm_nn(dy, w)
        dw = F.store_weight_grad(w, dy, x)
        return dx, dw, None


def linear_rs(x: torch.Tensor, w: torch.Tensor, group) -> torch.Tensor:
    """x [T, in_local], w [out, in_local] -> [T/n, out] (sum over ranks, scattered on rows)."""
    from ..ops import fused_comm
    if fused_comm.enabled(x, group):
        return fused_comm.linear_rs(x, w, group)
    return _LinearRS.apply(x, w, group)


# ----------------------------------------------------------------------------- ZeRO-3 linear


class Zero3Schedule:
    """Order of the ZeRO-3 weights of one model, used to prefetch the next gather.

    The reference gathers each weight synchronously right before its GEMM, forward and backward
    (reference ``utils/linear_zero3.py:35-43,62-65``), and names the missing overlap as a known
    cost (reference ``README.md:37``).  Here the weights register in forward order; while weight
    ``k`` is in use the gather of weight ``k+1`` (forward) or ``k-1`` (backward) runs on NCCL's
    stream into the other of two alternating buffers."""

    def __init__(self):
        self.weights: List[torch.Tensor] = []
        self.groups: List[object] = []
        self.enabled = True
        self.keep_gathered = False   # ZeRO-2 style: keep forward's gathered weights for backward
        self._inflight = {}    # index -> (tensor, work)
        self._kept = {}        # index -> gathered weight (keep_gathered only)

    def register(self, w: torch.Tensor, group) -> int:
        self.weights.append(w)
        self.groups.append(group)
        return len(self.weights) - 1

    def _launch(self, idx: int):
        w, group = self.weights[idx], self.groups[idx]
        n = C.group_size(group)
        buf = get_global_memory_buffer().get_tensor((n * w.shape[0],) + tuple(w.shape[1:]), w.dtype,
                                                    f"zero3_w{idx % 2}", w.device)
        full, work = C.all_gather_rows(w.detach(), group, out=buf, async_op=True)
        self._inflight[idx] = (full, work)

    def fetch(self, idx: int, direction: int) -> torch.Tensor:
        """Gathered weight ``idx``; starts the gather of ``idx + direction`` before returning."""
        if self.keep_gathered:
            # the reference's ``--use_zero2`` (FSDP SHARD_GRAD_OP, train.py:137-141): parameters stay
            # whole between forward and backward, trading memory for the second gather
            if direction < 0 and idx in self._kept:
                return self._kept.pop(idx)
            full = C.all_gather_rows(self.weights[idx].detach(), self.groups[idx])
            if direction > 0:
                self._kept[idx] = full
            return full
        if idx not in self._inflight:
            # a stale prefetch into the same slot must not be overwritten while in flight
            for j in [j for j in self._inflight if j % 2 == idx % 2]:
                _, wk = self._inflight.pop(j)
                if wk is not None:
                    wk.wait()
            self._launch(idx)
        full, work = self._inflight.pop(idx)
        if work is not None:
            work.wait()
        nxt = idx + direction
        if self.enabled and 0 <= nxt < len(self.weights) and nxt not in self._inflight \
                and self.weights[nxt].is_cuda and C.group_size(self.groups[nxt]) > 1:
            self._launch(nxt)
        return full

    def reset(self) -> None:
        for _, (_, wk) in list(self._inflight.items()):
            if wk is not None:
                wk.wait()
        self._inflight.clear()


class _Zero3Linear(Function):
    @staticmethod
    def forward(ctx, x, w, group, sched, idx):
        ctx.group, ctx.sched, ctx.idx = group, sched, idx
        ctx.save_for_backward(x, w)           # the SHARD is saved, never the gathered weight
        n = C.group_size(group)
        if n == 1:
            return F.gemm_nt(x, w)
        if sched is not None:
            full = sched.fetch(idx, +1)
        else:
            buf = get_global_memory_buffer().get_tensor((n * w.shape[0], w.shape[1]), w.dtype, "mpu", w.device)
            full = C.all_gather_rows(w, group, out=buf)
        return F.gemm_nt(x, full)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        group, sched, idx = ctx.group, ctx.sched, ctx.idx
        n = C.group_size(group)
        dy = dy.contiguous()
        if n == 1:
            dx = F.gemm_nn(dy, w) if ctx.needs_input_grad[0] else None
            return dx, F.store_weight_grad(w, dy, x), None, None, None
        if sched is not None:
            full = sched.fetch(idx, -1)
        else:
            buf = get_global_memory_buffer().get_tensor((n * w.shape[0], w.shape[1]), w.dtype, "mpu", w.device)
            full = C.all_gather_rows(w, group, out=buf)
        dx = F.gemm_nn(dy, full) if ctx.needs_input_grad[0] else None
        slot = f"zero3_g{idx % 2}"
        gfull = get_global_memory_buffer().get_tensor((n * w.shape[0], w.shape[1]), w.dtype, slot, w.device)
        # the previous reduce-scatter that read this slot must have drained
        prev = _SLOT_WORK.pop(slot, None)
        if prev is not None:
            prev.wait()
        F.gemm_tn(dy, x, out=gfull)
        mg = getattr(w, "main_grad", None)
        if mg is not None and not getattr(w, "_grad_written", False) and C._is_nccl(group):
            import torch.distributed as dist
            work = dist.reduce_scatter_tensor(mg, gfull, group=group, async_op=True)
            _SLOT_WORK[slot] = work
            _PENDING.append(work)
            w._grad_work = work
            w._grad_written = True
            dw = None
        else:
            # a second contribution to the same weight before the optimizer step: the reduce-scatter of the
            # first one may still be writing main_grad on NCCL's stream - finish it before accumulating
            first = getattr(w, "_grad_work", None)
            if first is not None:
                first.wait()
                w._grad_work = None
            dw = F.deliver_grad(w, C.reduce_scatter_rows(gfull, group))
        return dx, dw, None, None, None


_SLOT_WORK = {}


def zero3_linear(x: torch.Tensor, w_shard: torch.Tensor, group, sched: Optional[Zero3Schedule] = None,
                 idx: int = 0) -> torch.Tensor:
    """x [T, in] local tokens, w_shard [out/n, in] -> [T, out]."""
    from ..ops import fused_comm
    if fused_comm.enabled(x, group):
        return fused_comm.zero3_linear(x, w_shard, group, sched, idx)
    return _Zero3Linear.apply(x, w_shard, group, sched, idx)


class _Zero3Embedding(Function):
    @staticmethod
    def forward(ctx, ids, w, group):
        ctx.group = group
        ctx.save_for_backward(ids)
        ctx.w = w
        full = C.all_gather_rows(w, group)
        return full.index_select(0, ids)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        w, group = ctx.w, ctx.group
        n = C.group_size(group)
        g = torch.zeros((n * w.shape[0], w.shape[1]), dtype=dy.dtype if dy.is_cuda else torch.float32,
                        device=dy.device)
        g.index_add_(0, ids, dy.to(g.dtype))
        g = C.reduce_scatter_rows(g, group)
        return None, F.deliver_grad(w, g), None


def zero3_embedding(ids: torch.Tensor, w_shard: torch.Tensor, group) -> torch.Tensor:
    """Embedding lookup through a vocab-sharded table: gather, index, and reduce-scatter the
    scatter-added gradient (the reference leaves this to FSDP's flat parameter, train.py:114-159)."""
    return _Zero3Embedding.apply(ids, w_shard, group)


# ----------------------------------------------------------------------------- modules


class ColumnParallelLinearAG(nn.Module):
    """``[T/n, in] -> [T, out/n]``; weight ``[out/n, in]`` (this rank's rows of the full weight)."""

    def __init__(self, in_features: int, out_features_local: int, group, dtype=None, device=None):
        super().__init__()
        self.group = group
        self.weight = nn.Parameter(torch.empty(out_features_local, in_features, dtype=dtype, device=device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ag_linear(x, self.weight, self.group)

    def get_master_weight(self) -> torch.Tensor:
        """Full weight gathered over the group (reference ``get_master_weight``, linear_tpsp.py:474-477)."""
        return C.all_gather_rows(self.weight.detach(), self.group)


class RowParallelLinearRS(nn.Module):
    """``[T, in/n] -> [T/n, out]``; weight ``[out, in/n]`` (this rank's columns of the full weight)."""

    def __init__(self, in_features_local: int, out_features: int, group, dtype=None, device=None):
        super().__init__()
        self.group = group
        self.weight = nn.Parameter(torch.empty(out_features, in_features_local, dtype=dtype, device=device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear_rs(x, self.weight, self.group)

    def get_master_weight(self) -> torch.Tensor:
        parts = C.all_gather_rows(self.weight.detach().t().contiguous(), self.group)
        return parts.t().contiguous()


class LinearZeRO3(nn.Module):
    """``[T, in] -> [T, out]`` on local tokens; weight shard ``[out/n, in]``."""

    def __init__(self, in_features: int, out_features: int, group, sched: Optional[Zero3Schedule] = None,
                 dtype=None, device=None):
        super().__init__()
        n = C.group_size(group)
        if out_features % n:
            raise ValueError(f"ZeRO-3 linear: out_features {out_features} not divisible by group size {n}")
        self.group, self.sched = group, sched
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features // n, in_features, dtype=dtype, device=device))
        self.idx = sched.register(self.weight, group) if sched is not None else 0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return zero3_linear(x, self.weight, self.group, self.sched, self.idx)

    def get_master_weight(self) -> torch.Tensor:
        return C.all_gather_rows(self.weight.detach(), self.group)
