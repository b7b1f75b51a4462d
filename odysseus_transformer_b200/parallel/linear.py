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


class _GatherLastDim(Function):
    """[..., c] on each rank -> [..., n*c]; backward keeps this rank's slice (the reference's
    ``gather_from_model_parallel_region``, used for ``gather_output`` and ``get_master_weight``)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = C.group_size(group)
        if n == 1:
            return x
        parts = C.all_gather_rows(x.unsqueeze(0).contiguous(), group)           # [n, ..., c]
        return torch.cat(list(parts.unbind(0)), dim=-1)

    @staticmethod
    def backward(ctx, dy):
        n, r = C.group_size(ctx.group), C.group_rank(ctx.group)
        if n == 1:
            return dy, None
        c = dy.shape[-1] // n
        return dy[..., r * c:(r + 1) * c].contiguous(), None


class _ScatterLastDim(Function):
    """Keep this rank's slice of the last dim; backward all-gathers it (``input_is_parallel=False``)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n, r = C.group_size(group), C.group_rank(group)
        if n == 1:
            return x
        c = x.shape[-1] // n
        return x[..., r * c:(r + 1) * c].contiguous()

    @staticmethod
    def backward(ctx, dy):
        return _GatherLastDim.apply(dy, ctx.group), None


class _CopyToRegion(Function):
    """Identity forward, all-reduce backward: the input of a column-parallel linear that is NOT sequence parallel."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous().clone()
        C.all_reduce_(dy, ctx.group)
        return dy, None


class _ReduceFromRegion(Function):
    """All-reduce forward, identity backward: the output of a row-parallel linear that is NOT sequence parallel."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous().clone()
        C.all_reduce_(x, group)
        return x

    @staticmethod
    def backward(ctx, dy):
        return dy, None


def gather_last_dim(x: torch.Tensor, group) -> torch.Tensor:
    return _GatherLastDim.apply(x, group)


def scatter_last_dim(x: torch.Tensor, group) -> torch.Tensor:
    return _ScatterLastDim.apply(x, group)


# ----------------------------------------------------------------------------- AG -> GEMM (column parallel)


class _AGLinear(Function):
    @staticmethod
    def forward(ctx, x, w, group, rope=None):
        ctx.group = group
        ctx.save_for_backward(x, w)           # only the LOCAL shard of the input is kept
        n = C.group_size(group)
        if n == 1:
            return F.gemm_nt(x, w, rope=rope)
        buf = get_global_memory_buffer().get_tensor((n * x.shape[0], x.shape[1]), x.dtype, "mpu", x.device)
        total = C.all_gather_rows(x, group, out=buf)
        return F.gemm_nt(total, w, rope=rope)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        group = ctx.group
        n = C.group_size(group)
        dy = dy.contiguous()
        if n == 1:
            dx = F.gemm_nn(dy, w)
            return dx, F.store_weight_grad(w, dy, x), None, None
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
        return dx, dw, None, None


def ag_linear(x: torch.Tensor, w: torch.Tensor, group, rope=None) -> torch.Tensor:
    """x [T/n, in] (sequence shard), w [out_local, in] -> [T, out_local].

    ``rope`` (``ops.functional.RopeEpilogue``, tables for the T gathered rows): the product is a packed q|k|v
    projection and leaves the GEMM with its q / k heads rotated.  The op's backward still takes the gradient of the
    product BEFORE the rotation: whoever consumes the rotated product undoes the rotation on the gradient it returns
    (``parallel.attention.packed_rope_attention(..., pre_rotated=True)`` does)."""
    from ..ops import fused_comm
    if fused_comm.enabled(x, group):
        return fused_comm.ag_linear(x, w, group, rope)
    return _AGLinear.apply(x, w, group, rope)


# ----------------------------------------------------------------------------- GEMM -> RS (row parallel)


class _LinearRS(Function):
    @staticmethod
    def forward(ctx, x, w, group, residual=None):
        ctx.group = group
        ctx.save_for_backward(x, w)
        if C.group_size(group) == 1:
            return F.gemm_nt(x, w, residual=residual)
        y = C.reduce_scatter_rows(F.gemm_nt(x, w), group)
        return y if residual is None else y.add_(residual)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        n = C.group_size(ctx.group)
        dy = dy.contiguous()
        d_res = dy if ctx.needs_input_grad[3] else None      # the residual's gradient is the local rows' gradient itself
        if n > 1:
            buf = get_global_memory_buffer().get_tensor((n * dy.shape[0], dy.shape[1]), dy.dtype, "mpu", dy.device)
            dy = C.all_gather_rows(dy, ctx.group, out=buf)
        dx = F.gemm_nn(dy, w)
        dw = F.store_weight_grad(w, dy, x)
        return dx, dw, None, d_res


def linear_rs(x: torch.Tensor, w: torch.Tensor, group, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, in_local], w [out, in_local] -> [T/n, out] (sum over ranks, scattered on rows).

    ``residual`` [T/n, out]: added to this rank's rows where they are reduced (the residual stream joins the block's
    output in the producing kernel instead of in the next normalisation)."""
    from ..ops import fused_comm
    if fused_comm.enabled(x, group):
        return fused_comm.linear_rs(x, w, group, residual)
    return _LinearRS.apply(x, w, group, residual)


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
    def forward(ctx, x, w, group, sched, idx, rope=None, residual=None):
        ctx.group, ctx.sched, ctx.idx = group, sched, idx
        ctx.save_for_backward(x, w)           # the SHARD is saved, never the gathered weight
        n = C.group_size(group)
        if n == 1:
            return F.gemm_nt(x, w, rope=rope, residual=residual)
        if sched is not None:
            full = sched.fetch(idx, +1)
        else:
            buf = get_global_memory_buffer().get_tensor((n * w.shape[0], w.shape[1]), w.dtype, "mpu", w.device)
            full = C.all_gather_rows(w, group, out=buf)
        return F.gemm_nt(x, full, rope=rope, residual=residual)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        group, sched, idx = ctx.group, ctx.sched, ctx.idx
        n = C.group_size(group)
        dy = dy.contiguous()
        d_res = dy if ctx.needs_input_grad[6] else None
        if n == 1:
            dx = F.gemm_nn(dy, w) if ctx.needs_input_grad[0] else None
            return dx, F.store_weight_grad(w, dy, x), None, None, None, None, d_res
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
        return dx, dw, None, None, None, None, d_res


_SLOT_WORK = {}


def zero3_linear(x: torch.Tensor, w_shard: torch.Tensor, group, sched: Optional[Zero3Schedule] = None,
                 idx: int = 0, rope=None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, in] local tokens, w_shard [out/n, in] -> [T, out].  ``rope`` as in ``ag_linear`` (tables for the T local
    rows), ``residual`` [T, out] as in ``linear_rs``: both are applied in the GEMM epilogue."""
    from ..ops import fused_comm
    if fused_comm.enabled(x, group):
        return fused_comm.zero3_linear(x, w_shard, group, sched, idx, rope, residual)
    return _Zero3Linear.apply(x, w_shard, group, sched, idx, rope, residual)


class _Zero3Embedding(Function):
    """Lookup in a vocab-sharded table that moves only the rows the tokens touch.

    Token ids are sorted by owning rank and sent to the owners, which answer with their rows (two uneven
    all-to-alls of ``t`` ids and ``t x d`` values per rank); backward sends the output gradient rows back the
    same way and every owner scatter-adds them into its own shard in fp32.  Gathering the whole ``[V, d]``
    table and reduce-scattering a full-size gradient instead would move ``V x d`` twice per step (1 GB each way
    at Llama-3's vocabulary) and, with a bf16 scatter-add, lose precision on repeated token ids."""

    @staticmethod
    def forward(ctx, ids, w, group):
        n, r = C.group_size(group), C.group_rank(group)
        vr = w.shape[0]
        owner = torch.div(ids, vr, rounding_mode="floor")
        order = torch.argsort(owner, stable=True)
        counts = torch.bincount(owner, minlength=n)
        all_counts = C.all_gather_rows(counts.view(1, n), group).tolist()      # [source][owner]; one host read
        send = all_counts[r]
        recv = [all_counts[p][r] for p in range(n)]
        want = C.all_to_all_rows(ids[order], send, recv, group) - r * vr       # rows of my shard the others need
        rows = C.all_to_all_rows(w.detach().index_select(0, want), recv, send, group)
        out = torch.empty_like(rows)
        out[order] = rows
        ctx.group, ctx.w, ctx.send, ctx.recv = group, w, send, recv
        ctx.save_for_backward(order, want)
        return out

    @staticmethod
    def backward(ctx, dy):
        order, want = ctx.saved_tensors
        w = ctx.w
        got = C.all_to_all_rows(dy.index_select(0, order), ctx.send, ctx.recv, ctx.group)
        g = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        g.index_add_(0, want, got.float())
        return None, F.deliver_grad(w, g), None


def zero3_embedding(ids: torch.Tensor, w_shard: torch.Tensor, group) -> torch.Tensor:
    """Embedding lookup through a vocab-sharded table (the reference leaves the table to FSDP's flat
    parameter, train.py:114-159): ids go to the owning ranks, rows come back; gradients travel the same way."""
    return _Zero3Embedding.apply(ids, w_shard, group)


# ----------------------------------------------------------------------------- modules


class ColumnParallelLinearAG(nn.Module):
    """``[T/n, in] -> [T, out/n]``; weight ``[out/n, in]`` (this rank's rows of the full weight).

    Options of the reference's constructor (reference ``utils/linear_tpsp.py:405-500``): ``bias`` (this rank's
    ``out/n`` entries, zero-initialised, added after the GEMM), ``gather_output`` (all-gather the result on the
    feature dim -> ``[T, out]``), ``sequence_parallel=False`` (the input already holds the whole sequence: no
    gather; its gradient is all-reduced instead), ``keep_master_weight_for_test`` (``master_weight`` keeps the full
    ``[out, in]`` tensor this shard was cut from - set by ``init_from_master``).  The model blocks use the defaults:
    no bias, sharded output, sequence parallel."""

    def __init__(self, in_features: int, out_features_local: int, group, dtype=None, device=None, bias: bool = False,
                 gather_output: bool = False, sequence_parallel: bool = True, keep_master_weight_for_test: bool = False):
        super().__init__()
        self.group, self.gather_output, self.sequence_parallel = group, gather_output, sequence_parallel
        self.keep_master_weight_for_test = keep_master_weight_for_test
        self.master_weight: Optional[torch.Tensor] = None
        self.weight = nn.Parameter(torch.empty(out_features_local, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features_local, dtype=dtype, device=device)) if bias else None

    def init_from_master(self, master: torch.Tensor) -> None:
        """Fill this rank's shard from the full ``[out, in]`` weight (identical on every rank)."""
        r, rows = C.group_rank(self.group), self.weight.shape[0]
        with torch.no_grad():
            self.weight.copy_(master[r * rows:(r + 1) * rows])
        if self.keep_master_weight_for_test:
            self.master_weight = master.detach().clone()

    def forward(self, x: torch.Tensor, rope=None) -> torch.Tensor:
        """``rope``: see ``ag_linear``; only the sequence-parallel, bias-free form the model blocks use takes it."""
        if rope is not None and (not self.sequence_parallel or self.bias is not None or self.gather_output):
            raise ValueError("the rotary epilogue needs the sequence-parallel projection without bias or output gather")
        if self.sequence_parallel:
            y = ag_linear(x, self.weight, self.group, rope)
        else:
            y = F.linear(_CopyToRegion.apply(x, self.group), self.weight)
        if self.bias is not None:
            y = y + self.bias
        if self.gather_output:
            y = gather_last_dim(y, self.group)
        return y

    def get_master_weight(self) -> torch.Tensor:
        """Full weight gathered over the group (reference ``get_master_weight``, linear_tpsp.py:474-477)."""
        return C.all_gather_rows(self.weight.detach(), self.group)


class RowParallelLinearRS(nn.Module):
    """``[T, in/n] -> [T/n, out]``; weight ``[out, in/n]`` (this rank's columns of the full weight).

    Options of the reference's constructor (reference ``utils/linear_tpsp.py:503-596``): ``bias`` (full ``[out]``,
    zero-initialised, added after the reduction so it is counted once), ``input_is_parallel=False`` (the input
    holds all ``in`` features: this rank's slice is cut out first), ``sequence_parallel=False`` (all-reduce instead
    of reduce-scatter: every rank gets ``[T, out]``), ``keep_master_weight_for_test``.  Defaults as the model blocks
    use them: no bias, parallel input, sequence parallel."""

    def __init__(self, in_features_local: int, out_features: int, group, dtype=None, device=None, bias: bool = False,
                 input_is_parallel: bool = True, sequence_parallel: bool = True, keep_master_weight_for_test: bool = False):
        super().__init__()
        self.group, self.input_is_parallel, self.sequence_parallel = group, input_is_parallel, sequence_parallel
        self.keep_master_weight_for_test = keep_master_weight_for_test
        self.master_weight: Optional[torch.Tensor] = None
        self.weight = nn.Parameter(torch.empty(out_features, in_features_local, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        if self.bias is not None and C.group_size(group) > 1:
            # every rank adds the same bias to different rows (or, without sequence parallelism, to the same rows,
            # where each copy sees the full gradient): rows differ -> the gradients must be summed
            if sequence_parallel:
                self.bias.grad_sync_group = group

    def init_from_master(self, master: torch.Tensor) -> None:
        """Fill this rank's shard from the full ``[out, in]`` weight (identical on every rank)."""
        r, cols = C.group_rank(self.group), self.weight.shape[1]
        with torch.no_grad():
            self.weight.copy_(master[:, r * cols:(r + 1) * cols])
        if self.keep_master_weight_for_test:
            self.master_weight = master.detach().clone()

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual`` (this rank's output rows): added to the result, inside the kernel on the sequence-parallel path."""
        if not self.input_is_parallel:
            x = scatter_last_dim(x, self.group)
        if self.sequence_parallel:
            y = linear_rs(x, self.weight, self.group, residual if self.bias is None else None)
            if self.bias is not None and residual is not None:
                y = y + residual
        else:
            y = _ReduceFromRegion.apply(F.linear(x, self.weight), self.group)
            if residual is not None:
                y = y + residual
        if self.bias is not None:
            y = y + self.bias
        return y

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

    def forward(self, x: torch.Tensor, rope=None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        return zero3_linear(x, self.weight, self.group, self.sched, self.idx, rope, residual)

    def get_master_weight(self) -> torch.Tensor:
        return C.all_gather_rows(self.weight.detach(), self.group)
