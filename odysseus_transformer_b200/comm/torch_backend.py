"""Collectives over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).

This is the *baseline* data plane - the same collectives the reference issues
(reference ``utils/linear_tpsp.py:35-81``: reduce-scatter / all-gather along the first dim;
``utils/linear_zero3.py:41-43,82-84``: weight all-gather, gradient reduce-scatter with SUM) -
and the control plane for bootstrap.  A ``group`` of ``None`` or of size 1 turns every call into
the identity, so single-process runs share all code paths.

gloo has no reduce_scatter and no ``*_into_tensor`` forms on every build; those cases fall back to
list-based all-gather and all-reduce + slice, which keeps the CPU tests exact.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def group_size(group) -> int:
    if group is None or not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None or not dist.is_initialized():
        return 0
    return dist.get_rank(group)


def _is_nccl(group) -> bool:
    return dist.get_backend(group) == "nccl"


def all_gather_rows(x: torch.Tensor, group, out: Optional[torch.Tensor] = None, async_op: bool = False):
    """[t, ...] on each of n ranks -> [n*t, ...] (rank order). Returns tensor, or (tensor, work)."""
    n = group_size(group)
    if n == 1:
        return (x, None) if async_op else x
    x = x.contiguous()
    if out is None:
        out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if _is_nccl(group):
        work = dist.all_gather_into_tensor(out, x, group=group, async_op=async_op)
    else:
        parts = list(out.chunk(n, dim=0))
        work = dist.all_gather(parts, x, group=group, async_op=async_op)
    return (out, work) if async_op else out


def reduce_scatter_rows(x: torch.Tensor, group, async_op: bool = False):
    """[n*t, ...] partial sums on each rank -> [t, ...] summed slice of this rank."""
    n = group_size(group)
    if n == 1:
        return (x, None) if async_op else x
    x = x.contiguous()
    t = x.shape[0] // n
    if _is_nccl(group):
        out = torch.empty((t,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        work = dist.reduce_scatter_tensor(out, x, group=group, async_op=async_op)
        return (out, work) if async_op else out
    buf = x.clone()
    dist.all_reduce(buf, group=group)
    r = group_rank(group)
    out = buf[r * t:(r + 1) * t].clone()
    return (out, None) if async_op else out


def all_reduce_(x: torch.Tensor, group, async_op: bool = False):
    if group_size(group) == 1:
        return None
    return dist.all_reduce(x, group=group, async_op=async_op)


def all_to_all_chunks(x: torch.Tensor, group) -> torch.Tensor:
    """x [n, ...]: slice i goes to rank i; returns y [n, ...] with y[i] = slice sent by rank i."""
    n = group_size(group)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty_like(x)
    if _is_nccl(group):
        dist.all_to_all_single(out, x, group=group)
    else:
        ins = [t.contiguous() for t in x.unbind(0)]
        outs = [torch.empty_like(t) for t in ins]
        try:
            dist.all_to_all(outs, ins, group=group)
        except (RuntimeError, NotImplementedError):
            # transport without all-to-all: gather everything and pick
            gathered = [torch.empty_like(x) for _ in range(n)]
            dist.all_gather(gathered, x, group=group)
            r = group_rank(group)
            outs = [g[r] for g in gathered]
        out = torch.stack(outs, 0)
    return out


def all_to_all_rows(x: torch.Tensor, send_counts, recv_counts, group) -> torch.Tensor:
    """Uneven all-to-all on the first dim: rows [sum(send_counts[:p]), +send_counts[p]) of ``x`` go to rank p;
    returns the rows received, ordered by source rank (``recv_counts[p]`` rows from rank p).  Counts are host ints."""
    n = group_size(group)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((int(sum(recv_counts)),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(out, x, output_split_sizes=[int(c) for c in recv_counts],
                           input_split_sizes=[int(c) for c in send_counts], group=group)
    return out


def broadcast_(x: torch.Tensor, src_global_rank: int, group) -> None:
    if group_size(group) > 1:
        dist.broadcast(x, src=src_global_rank, group=group)


def barrier(group=None) -> None:
    if dist.is_initialized() and group_size(group if group is not None else dist.group.WORLD) > 1:
        dist.barrier(group=group)
