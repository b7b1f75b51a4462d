"""Inner x ring hybrid layouts (Ulysses x ring, Odysseus x ring).

The reference only claims these are possible (reference ``README.md:14``); they are specified here
by the mesh in ``mesh.py``: world = U (inner, adjacent ranks) x R (ring, strided ranks), sequence
zigzag-sharded over the ring dim and contiguously inside each ring block.  No new module is needed:
``SequenceParallelAttention`` (Ulysses) and ``TPSPAttention`` (Odysseus) both run their attention
core over ``ctx.ring_group``.  This file holds the helpers that pick degrees.
"""
from __future__ import annotations

from typing import Tuple


def choose_degrees(world_size: int, num_kv_heads: int, prefer_ring: int = 0) -> Tuple[int, int]:
    """Largest inner degree that divides the KV heads, rest goes to the ring (or ``prefer_ring``)."""
    if prefer_ring:
        if world_size % prefer_ring:
            raise ValueError(f"ring degree {prefer_ring} does not divide world size {world_size}")
        return world_size // prefer_ring, prefer_ring
    inner = 1
    for u in range(1, world_size + 1):
        if world_size % u == 0 and num_kv_heads % u == 0:
            inner = u
    return inner, world_size // inner


def describe(inner: int, ring: int) -> str:
    if ring == 1:
        return f"sp{inner}"
    if inner == 1:
        return f"ring{ring}"
    return f"sp{inner}xring{ring}"
