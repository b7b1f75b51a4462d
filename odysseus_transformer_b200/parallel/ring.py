"""Zigzag ring-attention mode.

The reference patches HF attention to call ``zigzag_ring_flash_attn_func`` with the default world
group (reference ``decoder/ring.py:10-39,99-114``).  Here ring mode is the ``inner degree 1`` corner
of the mesh: ``RingAttention`` is ``SequenceParallelAttention`` whose all-to-all is the identity and
whose attention core runs ``parallel.attention.zigzag_ring_attention`` over the ring group.
"""
from __future__ import annotations

from .attention import ring_attn_bwd, ring_attn_fwd, zigzag_ring_attention  # noqa: F401
from .ulysses import SequenceParallelAttention


class RingAttention(SequenceParallelAttention):
    def __init__(self, cfg, ctx, *a, **kw):
        if ctx.inner_size != 1:
            raise ValueError("ring mode uses inner degree 1; use the ulysses/odysseus hybrid for U > 1")
        super().__init__(cfg, ctx, *a, **kw)
