"""Timing, memory and JSON-lines metrics.

The reference prints allocated / reserved GB and the loss on rank 0 and sums ``time.time()`` deltas
over the steps after warm-up with no device synchronisation (reference ``train.py:104-107,185-186,
217-229,237-240``).  The same prints are kept by ``train``; this module adds what they lack:
device-side timing (CUDA events) reduced as the **max over ranks**, peak memory, exposed communication
time, per-phase timers and a JSONL sink.
"""
from __future__ import annotations

import json
import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class DeviceTimer:
    """Times a region on the current CUDA stream with events; wall clock on CPU."""

    def __init__(self, device: torch.device):
        self.cuda = device.type == "cuda"
        self.device = device
        self._pairs: List = []
        self._t0 = None
        self._cpu_ms = 0.0

    def start(self) -> None:
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._t0 = e
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> None:
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._pairs.append((self._t0, e))
        else:
            self._cpu_ms += (time.perf_counter() - self._t0) * 1e3

    def elapsed_ms(self) -> float:
        if self.cuda:
            torch.cuda.synchronize(self.device)
            return float(sum(a.elapsed_time(b) for a, b in self._pairs))
        return self._cpu_ms


def max_over_ranks(value: float, device: torch.device, group=None) -> float:
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device if device.type == "cuda" else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def memory_gb(device: torch.device) -> Dict[str, float]:
    if device.type != "cuda":
        return {"allocated": 0.0, "reserved": 0.0, "peak_allocated": 0.0, "peak_reserved": 0.0}
    g = 1024 ** 3
    return {"allocated": torch.cuda.memory_allocated(device) / g, "reserved": torch.cuda.memory_reserved(device) / g,
            "peak_allocated": torch.cuda.max_memory_allocated(device) / g,
            "peak_reserved": torch.cuda.max_memory_reserved(device) / g}


def exposed_comm_ms(ctx, reset: bool = False) -> float:
    """Communication time the step could not hide, in ms, max over ranks, since the last reset.

    The fused kernels time their own waits on other GPUs (``ody_set_wait_accumulator``): the TMA
    producer of every gather-GEMM CTA while remote rows have not arrived, one thread per
    reduce-scatter CTA while the other sources' tiles are missing, and the stand-alone wait kernels
    of the ring and Ulysses paths (during which the stream does nothing else).  The first two are
    summed over CTAs on the device and divided by the SM count here - the mean time an SM sat idle
    for data; the third counts in full.  0.0 without a symmetric heap (NCCL composition: the
    collectives are separate kernels and their cost is visible in the profiler instead).  Synchronises."""
    acc = getattr(ctx, "wait_acc", None)
    if acc is None:
        return 0.0
    v = acc.tolist()
    if reset:
        acc.zero_()
    sms = torch.cuda.get_device_properties(ctx.device).multi_processor_count
    ms = (v[0] + v[1]) / max(1, sms) / 1e6 + v[2] / 1e6
    return max_over_ranks(ms, ctx.device, ctx.world_group)


class PhaseTimers:
    """Named CUDA-event timers (forward / backward / optimizer ...) summed per phase; ``summary`` reduces
    every phase as the max over ranks.  On CPU it falls back to wall clock."""

    def __init__(self, device: torch.device):
        self.device = device
        self.timers: Dict[str, DeviceTimer] = {}

    def phase(self, name: str):
        import contextlib

        @contextlib.contextmanager
        def cm():
            t = self.timers.setdefault(name, DeviceTimer(self.device))
            t.start()
            try:
                yield
            finally:
                t.stop()
        return cm()

    def summary(self, group=None) -> Dict[str, float]:
        return {k: max_over_ranks(t.elapsed_ms(), self.device, group) for k, t in sorted(self.timers.items())}


class JsonlWriter:
    def __init__(self, path: Optional[str], rank: int = 0):
        self.f = open(path, "a") if (path and rank == 0) else None

    def write(self, **rec) -> None:
        if self.f is not None:
            self.f.write(json.dumps(rec) + "\n")
            self.f.flush()

    def close(self) -> None:
        if self.f is not None:
            self.f.close()
            self.f = None


def train_flops_per_token(cfg, seq_len: int) -> float:
    """Model FLOPs per trained token (fwd + bwd = 3x fwd), causal attention counted at half."""
    d, i = cfg.hidden_size, cfg.intermediate_size
    lin = 2 * (d * cfg.q_size + 2 * d * cfg.kv_size + cfg.q_size * d + 3 * d * i)
    attn = 2 * 2 * seq_len * cfg.q_size / 2
    head = 2 * d * cfg.vocab_size
    return 3.0 * (cfg.num_hidden_layers * (lin + attn) + head)
