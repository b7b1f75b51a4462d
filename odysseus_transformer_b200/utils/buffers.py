"""Named grow-only scratch buffers.

Same role as the reference's ``GlobalMemoryBuffer`` (reference ``utils/globals.py:9-41``): gathered
activations and gathered weights are written into a cached flat tensor keyed by ``(name, dtype)``
instead of a fresh allocation per call, so nothing gathered outlives the next gather into the same
name and the allocator never fragments on these large temporaries.  Unlike the reference there are
several names (activations, and two alternating weight slots for prefetch), because a prefetched
weight must survive the activation gather that runs meanwhile.
"""
from __future__ import annotations

from functools import reduce
import operator
from typing import Dict, Optional, Tuple

import torch


class GlobalMemoryBuffer:
    def __init__(self, device=None):
        self.device = device
        self._buf: Dict[Tuple[str, torch.dtype, str], torch.Tensor] = {}

    def get_tensor(self, shape, dtype: torch.dtype, name: str, device=None) -> torch.Tensor:
        device = torch.device(device if device is not None else (self.device or "cpu"))
        n = reduce(operator.mul, shape, 1)
        key = (name, dtype, str(device))
        cur = self._buf.get(key)
        if cur is None or cur.numel() < n:
            self._buf[key] = cur = torch.empty(n, dtype=dtype, device=device)
        return cur[:n].view(*shape)

    def bytes_held(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._buf.values())

    def clear(self) -> None:
        self._buf.clear()


_GLOBAL: Optional[GlobalMemoryBuffer] = None


def set_global_memory_buffer(device=None) -> GlobalMemoryBuffer:
    """(Re)create the process-wide buffer (reference ``_set_global_memory_buffer``)."""
    global _GLOBAL
    _GLOBAL = GlobalMemoryBuffer(device)
    return _GLOBAL


def get_global_memory_buffer() -> GlobalMemoryBuffer:
    global _GLOBAL
    if _GLOBAL is None:
        _GLOBAL = GlobalMemoryBuffer()
    return _GLOBAL
