"""Profiling hooks.

``init_prof`` keeps the reference's contract (reference ``train.py:28-46``): a ``torch.profiler``
context with CUDA activity, schedule wait=0 / warmup=2 / active=4 / repeat=1 and a TensorBoard
trace handler writing to ``./profile/``, or a ``nullcontext`` whose ``step()`` is never called.
``nvtx_range`` marks the fused paths for timeline tools.
"""
from __future__ import annotations

import contextlib
from contextlib import nullcontext

import torch


def init_prof(use_profiler: bool, out_dir: str = "./profile/"):
    if not use_profiler:
        return nullcontext()
    activities = [torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() \
        else [torch.profiler.ProfilerActivity.CPU]
    return torch.profiler.profile(
        activities=activities,
        schedule=torch.profiler.schedule(wait=0, warmup=2, active=4, repeat=1),
        on_trace_ready=torch.profiler.tensorboard_trace_handler(out_dir),
        record_shapes=True,
        with_stack=True,
    )


@contextlib.contextmanager
def nvtx_range(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield
