"""Process mesh and sequence-sharding index maths.

The reference has a single model-parallel group equal to the whole world, created through
fairscale (reference ``train.py:58-60``), and slices inputs contiguously or in zigzag order
(reference ``utils/apply_seq_parallel.py:4-12,93-98``).  This module owns both: a
``ParallelContext`` describing a 2-D mesh ``inner (Ulysses / Odysseus / TP-SP degree U) x
ring (zigzag ring degree R)`` with ``world = U * R``, and the index functions that say which
global token positions live on which rank.

Rank layout: ``rank = ring_rank * U + inner_rank`` - inner-group peers are adjacent ranks.

Sequence layout (global length ``L``):
  * the sequence is cut into ``2R`` chunks; ring rank ``j`` owns chunks ``j`` and ``2R-1-j``
    (zigzag, so every ring rank does the same amount of causal attention work);
  * that *ring block* of ``L/R`` tokens is cut contiguously into ``U`` pieces; inner rank ``u``
    owns piece ``u`` (``L/N`` tokens).
With ``R == 1`` this is the plain contiguous shard of Ulysses / Odysseus / TP-SP, with
``U == 1`` it is the zigzag shard of ring attention.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist


def zigzag_block_indices(seq_len: int, ring_size: int, ring_rank: int) -> torch.Tensor:
    """Global positions of the ring block of ``ring_rank`` (chunks j and 2R-1-j), in local order."""
    if seq_len % (2 * ring_size) != 0:
        raise ValueError(f"seq_len {seq_len} must be divisible by 2*ring_size={2 * ring_size}")
    c = seq_len // (2 * ring_size)
    lo = torch.arange(ring_rank * c, (ring_rank + 1) * c)
    hi_chunk = 2 * ring_size - 1 - ring_rank
    hi = torch.arange(hi_chunk * c, (hi_chunk + 1) * c)
    return torch.cat([lo, hi])


def block_indices(seq_len: int, ring_size: int, ring_rank: int) -> torch.Tensor:
    if ring_size == 1:
        return torch.arange(seq_len)
    return zigzag_block_indices(seq_len, ring_size, ring_rank)


def local_indices(seq_len: int, inner_size: int, ring_size: int, inner_rank: int, ring_rank: int) -> torch.Tensor:
    """Global positions of the ``L/N`` tokens owned by mesh coordinate (ring_rank, inner_rank)."""
    blk = block_indices(seq_len, ring_size, ring_rank)
    if blk.numel() % inner_size != 0:
        raise ValueError(f"ring block of {blk.numel()} tokens not divisible by inner degree {inner_size}")
    t = blk.numel() // inner_size
    return blk[inner_rank * t:(inner_rank + 1) * t]


@dataclass
class ParallelContext:
    """Everything a parallel module needs to know about where it runs."""

    rank: int = 0
    world_size: int = 1
    inner_size: int = 1
    ring_size: int = 1
    device: torch.device = field(default_factory=lambda: torch.device("cpu"))
    world_group: Optional[object] = None
    inner_group: Optional[object] = None
    ring_group: Optional[object] = None
    backend: str = "library"       # "library": torch ops + torch.distributed ; "fused": sm_100a kernels
    symm: Optional[object] = None  # symmetric-memory heap (comm.symm.SymmetricHeap) when peer access is set up
    wait_acc: Optional[torch.Tensor] = None   # int64[4] device totals (ns) of the fused kernels' waits on other GPUs

    @property
    def inner_rank(self) -> int:
        return self.rank % self.inner_size

    @property
    def ring_rank(self) -> int:
        return self.rank // self.inner_size

    @property
    def inner_ranks(self) -> List[int]:
        base = self.ring_rank * self.inner_size
        return list(range(base, base + self.inner_size))

    @property
    def ring_ranks(self) -> List[int]:
        return [j * self.inner_size + self.inner_rank for j in range(self.ring_size)]

    @property
    def is_distributed(self) -> bool:
        return self.world_size > 1

    def local_indices(self, seq_len: int) -> torch.Tensor:
        return local_indices(seq_len, self.inner_size, self.ring_size, self.inner_rank, self.ring_rank)

    def block_indices(self, seq_len: int) -> torch.Tensor:
        return block_indices(seq_len, self.ring_size, self.ring_rank)

    def check_model(self, cfg, mode: str) -> None:
        """Divisibility rules of each mode (reference decoder/odysseus.py:76-77 needs N | Hkv)."""
        U = self.inner_size
        if mode in ("odysseus", "tpsp", "ulysses") and U > 1:
            if cfg.num_attention_heads % U or cfg.num_key_value_heads % U:
                raise ValueError(
                    f"mode {mode}: inner degree {U} must divide heads {cfg.num_attention_heads} "
                    f"and kv heads {cfg.num_key_value_heads}")
        if mode == "tpsp" and cfg.intermediate_size % U:
            raise ValueError(f"tpsp: inner degree {U} must divide intermediate size {cfg.intermediate_size}")


_CTX: Optional[ParallelContext] = None


def get_context() -> ParallelContext:
    global _CTX
    if _CTX is None:
        _CTX = ParallelContext()
    return _CTX


def set_context(ctx: Optional[ParallelContext]) -> None:
    global _CTX
    _CTX = ctx


def mode_degrees(mode: Optional[str], world_size: int, ulysses_degree: int = 0, ring_degree: int = 1):
    """(inner, ring) degrees implied by a parallel mode and the optional hybrid flags."""
    if mode in (None, "dp"):
        return 1, 1
    if mode == "ring":
        if ulysses_degree not in (0, 1):
            raise ValueError("ring mode is the U=1 corner of the mesh; use ulysses/odysseus with --ring-degree for a hybrid")
        return 1, world_size
    ring = max(1, ring_degree)
    inner = ulysses_degree if ulysses_degree > 0 else world_size // ring
    if inner * ring != world_size:
        raise ValueError(f"inner degree {inner} x ring degree {ring} != world size {world_size}")
    if mode == "tpsp" and ring != 1:
        raise ValueError("tpsp has no ring hybrid (its MLP gathers the sequence across the whole group)")
    return inner, ring


def init_parallel_context(
    mode: Optional[str] = None,
    ulysses_degree: int = 0,
    ring_degree: int = 1,
    device: Optional[torch.device] = None,
    backend: str = "auto",
    timeout_s: float = 600.0,
) -> ParallelContext:
    """Build the mesh for ``mode`` on top of an initialised (or absent) default process group.

    If torch.distributed is not initialised and the torchrun environment variables are present,
    it is initialised here (NCCL for CUDA devices, gloo otherwise) - the analogue of the reference's
    ``dist.init_process_group("nccl")`` + ``initialize_model_parallel`` (train.py:56-60).
    """
    if device is None:
        if torch.cuda.is_available():
            local_rank = int(os.environ.get("LOCAL_RANK", 0))
            torch.cuda.set_device(local_rank)
            device = torch.device("cuda", local_rank)
        else:
            device = torch.device("cpu")
    if not dist.is_initialized() and "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        kw = {}
        if device.type == "cuda":
            kw["device_id"] = device
        dist.init_process_group(
            backend="nccl" if device.type == "cuda" else "gloo",
            timeout=datetime.timedelta(seconds=timeout_s), **kw)
    if dist.is_initialized():
        rank, world = dist.get_rank(), dist.get_world_size()
    else:
        rank, world = 0, 1
    inner, ring = mode_degrees(mode, world, ulysses_degree, ring_degree)
    if mode in (None, "dp"):
        inner, ring = 1, 1
    if backend == "auto":
        backend = "fused" if device.type == "cuda" else "library"
    ctx = ParallelContext(rank=rank, world_size=world, inner_size=inner, ring_size=ring,
                          device=device, backend=backend)
    if world > 1:
        ctx.world_group = dist.group.WORLD
        ctx.inner_group, ctx.ring_group = _make_groups(rank, world, inner, ring, timeout_s)
    set_context(ctx)
    return ctx


def _make_groups(rank: int, world: int, inner: int, ring: int, timeout_s: float):
    """Create inner (adjacent ranks) and ring (strided ranks) groups; every rank creates all of them."""
    timeout = datetime.timedelta(seconds=timeout_s)
    inner_group = ring_group = None
    if inner == world:
        inner_group = dist.group.WORLD
    elif inner > 1:
        for j in range(ring):
            ranks = list(range(j * inner, (j + 1) * inner))
            g = dist.new_group(ranks, timeout=timeout)
            if rank in ranks:
                inner_group = g
    if ring == world:
        ring_group = dist.group.WORLD
    elif ring > 1:
        for u in range(inner):
            ranks = [j * inner + u for j in range(ring)]
            g = dist.new_group(ranks, timeout=timeout)
            if rank in ranks:
                ring_group = g
    return inner_group, ring_group
