"""Timing, memory and JSON-lines metrics.

The reference prints allocated / reserved GB and the loss on rank 0 and sums ``time.time()`` deltas
over the steps after warm-up with no device synchronisation (reference ``train.py:104-107,185-186,
217-229,237-240``).  The same prints are kept by ``train``; this module adds what they lack:
device-side timing (CUDA events) reduced as the **max over ranks**, peak memory, and a JSONL sink.
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
