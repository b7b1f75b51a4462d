"""Symmetric peer-memory heap for the fused compute+collective kernels.

Each rank allocates one identical buffer through ``torch.distributed._symmetric_memory`` and exchanges
handles once; afterwards every rank holds the peers' base pointers, so kernels load from / store to peer
HBM over NVLink directly.  The reference moves all data with NCCL collectives through
``torch.distributed`` (reference ``utils/linear_tpsp.py:35-81``, ``utils/linear_zero3.py:41-43,82-84``);
here NCCL remains the bootstrap and the fallback, and this heap is the data plane of ``ops.fused_comm``.

Layout: ``[flag words (epochs and counters written by peers) | data]``.  Data is handed out by a bump
allocator; since every rank performs the same allocations in the same order, offsets agree everywhere.
*Slots* bundle what one fused call site needs:

* ``GatherSlot``  - a gathered buffer ``[n * chunk_rows, cols]`` that every rank pushes its shard into, plus
  per-row-block arrival counters, per-source completion counters and ``free`` epoch words;
* ``ScatterSlot`` - staging ``[n (source), chunk_rows, cols]`` plus ``arrived`` counters and ``consumed``
  epoch words.

Slots are keyed by shape and come in pairs used alternately, so a rank that is one call ahead of a peer
writes into the other buffer instead of waiting for the peer to drain the first.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

FLAG_BYTES = 1 << 20
ALIGN = 1024


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class GatherSlot:
    def __init__(self, heap: "SymmetricHeap", chunk_rows: int, cols: int):
        n = heap.n
        self.heap, self.chunk_rows, self.cols = heap, chunk_rows, cols
        self.buf_off = heap.alloc(n * chunk_rows * cols * 2)
        unit = 128 if chunk_rows % 128 == 0 else 64        # must match the kernel launcher's choice
        self.flags_off = heap.alloc_flags(n * (chunk_rows // unit))   # arrival counters, written by the pushers
        self.counters_off = heap.alloc_flags(n)                        # whole-shard counters, one per source
        self.free_off = heap.alloc_flags(n)                            # epochs written by the consumers
        self.gemm_done = torch.zeros(1, dtype=torch.int32, device=heap.device)
        self.uses = 0            # epoch: number of pushes into this buffer so far
        self.push_total = 0      # CTAs that have pushed into it (sum over uses)
        self.consume_total = 0   # CTAs that have consumed it (sum over uses)

    def view(self) -> torch.Tensor:
        """This rank's gathered buffer as a ``[n * chunk_rows, cols]`` bf16 tensor."""
        return self.heap.view(self.buf_off, (self.heap.n * self.chunk_rows, self.cols), torch.bfloat16)

    def _common(self, n_cta: int) -> Dict:
        h = self.heap
        return {"n_ranks": h.n, "rank": h.rank, "chunk_rows": self.chunk_rows, "cols": self.cols, "n_cta": n_cta,
                "epoch": self.uses, "prev_epoch": self.uses - 1, "uses": self.uses,
                "push_total": self.push_total, "consume_total": self.consume_total,
                "gathered_ptrs": [h.ptr(p, self.buf_off) for p in range(h.n)],
                "flags_ptrs": [h.ptr(p, self.flags_off) for p in range(h.n)],
                "counters_ptrs": [h.ptr(p, self.counters_off) for p in range(h.n)],
                "free_ptrs": [h.ptr(p, self.free_off) for p in range(h.n)],
                "gemm_done": self.gemm_done, "stats": h.stats}

    def push_desc(self, shard: torch.Tensor, n_cta: int) -> Dict:
        """Start a new epoch of this buffer: ``n_cta`` CTAs (of a GEMM launch or of ``push_shard``) will
        deliver ``shard`` into every rank's copy.  All ranks must make the same call."""
        self.uses += 1
        self.push_total += n_cta
        d = self._common(n_cta)
        d["shard"] = shard
        return d

    def consume_desc(self, which: int, n_cta: int) -> Dict:
        """A GEMM of ``n_cta`` CTAs reads the current epoch as operand ``which`` (1 = A, 2 = B)."""
        self.consume_total += n_cta
        d = self._common(n_cta)
        d["which"] = which
        return d


class ScatterSlot:
    def __init__(self, heap: "SymmetricHeap", chunk_rows: int, cols: int):
        n = heap.n
        self.heap, self.chunk_rows, self.cols = heap, chunk_rows, cols
        self.stage_off = heap.alloc(n * chunk_rows * cols * 2)
        self.arrived_off = heap.alloc_flags(n)
        self.consumed_off = heap.alloc_flags(n)
        self.reduce_counter = torch.zeros(1, dtype=torch.int32, device=heap.device)
        self.uses = 0
        self.arrived_total = 0
        # tiles (128 rows x 256 columns) of the full [n * chunk_rows, cols] product that touch this rank's rows
        M, r = n * chunk_rows, heap.rank
        lo, hi = r * chunk_rows, min((r + 1) * chunk_rows, M) - 1
        self.tiles_per_use = (hi // 128 - lo // 128 + 1) * ((cols + 255) // 256)

    def describe(self, out: torch.Tensor) -> Dict:
        h = self.heap
        self.uses += 1
        self.arrived_total += self.tiles_per_use
        return {"n_ranks": h.n, "rank": h.rank, "chunk_rows": self.chunk_rows, "epoch": self.uses,
                "prev_epoch": self.uses - 1, "uses": self.uses, "arrived_target": self.arrived_total, "out": out,
                "stage_ptrs": [h.ptr(p, self.stage_off) for p in range(h.n)],
                "arrived_ptrs": [h.ptr(p, self.arrived_off) for p in range(h.n)],
                "consumed_ptrs": [h.ptr(p, self.consumed_off) for p in range(h.n)],
                "reduce_counter": self.reduce_counter}


class InboxSlot:
    """Per-source inboxes ``[n (source), rows, cols]`` that peers fill with their own kernels' output stores
    (ring attention backward: the dK/dV a rank computes for another rank's keys), with one ``arrived`` epoch
    word per source and one ``consumed`` epoch word per owner."""

    def __init__(self, heap: "SymmetricHeap", rows: int, cols: int):
        n = heap.n
        self.heap, self.rows, self.cols = heap, rows, cols
        self.buf_off = heap.alloc(n * rows * cols * 2)
        self.arrived_off = heap.alloc_flags(n)
        self.consumed_off = heap.alloc_flags(n)
        self.uses = 0

    def begin(self) -> int:
        self.uses += 1
        return self.uses

    def local(self) -> torch.Tensor:
        return self.heap.view(self.buf_off, (self.heap.n, self.rows, self.cols), torch.bfloat16)

    def on_peer(self, peer: int) -> torch.Tensor:
        """Rank ``peer``'s inboxes as a tensor over its memory: only for this package's own kernels to store into."""
        return self.heap.peer_view(peer, self.buf_off, (self.heap.n, self.rows, self.cols), torch.bfloat16)

    def arrived_local(self) -> int:
        return self.heap.ptr(self.heap.rank, self.arrived_off)

    def consumed_local(self) -> int:
        return self.heap.ptr(self.heap.rank, self.consumed_off)

    def arrived_ptrs(self) -> List[int]:
        return [self.heap.ptr(p, self.arrived_off) for p in range(self.heap.n)]

    def consumed_ptrs(self) -> List[int]:
        return [self.heap.ptr(p, self.consumed_off) for p in range(self.heap.n)]


class A2ASlot:
    """Receive buffer ``[rows, cols]`` of an all-to-all whose senders are kernels (a GEMM epilogue or an
    attention epilogue storing straight into the destination), with one ``arrived`` word per source and
    one ``consumed`` epoch word per destination.  GEMM senders count CTAs into ``arrived`` (cumulative
    target); stream-ordered senders set it to the epoch."""

    def __init__(self, heap: "SymmetricHeap", rows: int, cols: int):
        n = heap.n
        self.heap, self.rows, self.cols = heap, rows, cols
        self.buf_off = heap.alloc(rows * cols * 2)
        self.arrived_off = heap.alloc_flags(n)
        self.consumed_off = heap.alloc_flags(n)
        self.uses = 0
        self.arrived_total = 0
        self._dummy = torch.zeros(1, dtype=torch.int32, device=heap.device)

    def local(self) -> torch.Tensor:
        return self.heap.view(self.buf_off, (self.rows, self.cols), torch.bfloat16)

    def on_peer(self, peer: int) -> torch.Tensor:
        """Rank ``peer``'s receive buffer: only for this package's own kernels to store into."""
        return self.heap.peer_view(peer, self.buf_off, (self.rows, self.cols), torch.bfloat16)

    def begin_epoch(self) -> int:
        self.uses += 1
        self.arrived_total = self.uses
        return self.uses

    def gemm_desc(self, a2a_cols: int, row0: int, col0: int, n_cta: int) -> Dict:
        """Scatter description (mode 2) for ``gemm_comm``: column group ``o`` of the product goes to rank ``o``'s
        buffer at rows ``row0 + r`` and columns ``col0 + c``; every one of the ``n_cta`` CTAs reports once."""
        h = self.heap
        self.uses += 1
        self.arrived_total += n_cta
        return {"mode": 2, "n_ranks": h.n, "rank": h.rank, "chunk_rows": 0, "epoch": self.uses, "prev_epoch": self.uses - 1,
                "uses": self.uses, "arrived_target": self.arrived_total, "out": self.local(),
                "stage_ptrs": [h.ptr(p, self.buf_off) for p in range(h.n)],
                "arrived_ptrs": self.arrived_ptrs(), "consumed_ptrs": self.consumed_ptrs(),
                "reduce_counter": self._dummy, "a2a_cols": a2a_cols, "a2a_ld": self.cols, "a2a_row0": row0, "a2a_col0": col0}

    def arrived_local(self) -> int:
        return self.heap.ptr(self.heap.rank, self.arrived_off)

    def consumed_local(self) -> int:
        return self.heap.ptr(self.heap.rank, self.consumed_off)

    def arrived_ptrs(self) -> List[int]:
        return [self.heap.ptr(p, self.arrived_off) for p in range(self.heap.n)]

    def consumed_ptrs(self) -> List[int]:
        return [self.heap.ptr(p, self.consumed_off) for p in range(self.heap.n)]


class SymmetricHeap:
    def __init__(self, group, device: torch.device, data_bytes: int):
        import torch.distributed._symmetric_memory as symm_mem
        self.group, self.device = group, device
        self.n = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self.capacity = _round_up(data_bytes, ALIGN)
        total = FLAG_BYTES + self.capacity
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:  # noqa: BLE001  (newer torch enables groups implicitly)
            pass
        self.local = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.local, group)
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self.local[:FLAG_BYTES].zero_()
        if os.environ.get("ODY_POISON_HEAP", "0") == "1":
            # debug aid: staging that is read before its data arrived then shows up as NaN in the result
            from ..utils.debug import poison_
            poison_(self.local[FLAG_BYTES:].view(torch.bfloat16))
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        self._data_top = 0
        self._flag_top = 0
        self._side: Optional[torch.cuda.Stream] = None
        self._peer_bufs: Dict[int, torch.Tensor] = {}
        self._inbox: Dict[Tuple[int, int], List[InboxSlot]] = {}
        self._a2a: Dict[Tuple[int, int, str], List[A2ASlot]] = {}
        self._gather: Dict[Tuple[int, int, str], List[GatherSlot]] = {}
        self._scatter: Dict[Tuple[int, int], List[ScatterSlot]] = {}
        self._toggle: Dict[Tuple[str, int, int], int] = {}
        # optional per-CTA timeline of the last gather launch (set by enable_stats)
        self.stats: Optional[torch.Tensor] = None

    def enable_stats(self) -> torch.Tensor:
        """Have gather GEMMs record, per CTA, [comm begin, comm end, producer wait for rows, CTA end] in ns."""
        self.stats = torch.zeros(self.sm_count * 4, dtype=torch.int64, device=self.device)
        return self.stats

    # ---- raw allocation (identical sequence on every rank)
    def alloc(self, nbytes: int) -> Optional[int]:
        nbytes = _round_up(nbytes, ALIGN)
        if self._data_top + nbytes > self.capacity:
            raise MemoryError("symmetric heap exhausted")
        off = FLAG_BYTES + self._data_top
        self._data_top += nbytes
        return off

    def alloc_flags(self, nwords: int) -> int:
        nbytes = _round_up(nwords * 4, 128)
        if self._flag_top + nbytes > FLAG_BYTES:
            raise MemoryError("symmetric flag area exhausted")
        off = self._flag_top
        self._flag_top += nbytes
        return off

    def ptr(self, peer: int, off: int) -> int:
        return self.ptrs[peer] + off

    def view(self, off: int, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.local[off:off + nbytes].view(dtype).view(*shape)

    def peer_view(self, peer: int, off: int, shape, dtype: torch.dtype) -> torch.Tensor:
        """A tensor over rank ``peer``'s copy of the heap.  Hand it only to this package's own kernels
        (plain or TMA stores / non-multicast loads); never to a library op."""
        if peer == self.rank:
            return self.view(off, shape, dtype)
        if peer not in self._peer_bufs:
            self._peer_bufs[peer] = self.handle.get_buffer(peer, (FLAG_BYTES + self.capacity,), torch.uint8, 0)
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self._peer_bufs[peer][off:off + nbytes].view(dtype).view(*shape)

    def inbox_slot(self, rows: int, cols: int) -> Optional[InboxSlot]:
        key = (rows, cols)
        if key not in self._inbox:
            if cols % 8 or not self.can_hold(self.n * rows * cols * 2):
                return None
            self._inbox[key] = [InboxSlot(self, rows, cols), InboxSlot(self, rows, cols)]
        t = self._toggle.get(("i",) + key, 0)
        self._toggle[("i",) + key] = t ^ 1
        return self._inbox[key][t]

    def a2a_slot(self, rows: int, cols: int, tag: str = "") -> Optional[A2ASlot]:
        key = (rows, cols, tag)
        if key not in self._a2a:
            if cols % 64 or not self.can_hold(rows * cols * 2):
                return None
            self._a2a[key] = [A2ASlot(self, rows, cols), A2ASlot(self, rows, cols)]
        t = self._toggle.get(("a",) + key, 0)
        self._toggle[("a",) + key] = t ^ 1
        return self._a2a[key][t]

    def can_hold(self, nbytes: int) -> bool:
        return self._data_top + _round_up(nbytes, ALIGN) * 2 <= self.capacity

    # ---- slots
    def side_stream(self) -> torch.cuda.Stream:
        """A second stream of this device for push-only launches that overlap compute."""
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        return self._side

    def gather_slot(self, chunk_rows: int, cols: int, tag: str = "") -> Optional[GatherSlot]:
        """``tag`` separates call sites whose flag protocols differ (ring attention never raises the
        row-block counters of a rank's own rows) from the GEMM gathers of the same shape."""
        key = (chunk_rows, cols, tag)
        if key not in self._gather:
            if chunk_rows % 64 or cols % 64 or not self.can_hold(self.n * chunk_rows * cols * 2):
                return None
            self._gather[key] = [GatherSlot(self, chunk_rows, cols), GatherSlot(self, chunk_rows, cols)]
        t = self._toggle.get(("g",) + key, 0)
        self._toggle[("g",) + key] = t ^ 1
        return self._gather[key][t]

    def scatter_slot(self, chunk_rows: int, cols: int) -> Optional[ScatterSlot]:
        key = (chunk_rows, cols)
        if key not in self._scatter:
            if cols % 8 or not self.can_hold(self.n * chunk_rows * cols * 2):
                return None
            self._scatter[key] = [ScatterSlot(self, chunk_rows, cols), ScatterSlot(self, chunk_rows, cols)]
        t = self._toggle.get(("s",) + key, 0)
        self._toggle[("s",) + key] = t ^ 1
        return self._scatter[key][t]


def heap_bytes_estimate(cfg, tokens_per_rank: int, n: int, ring: bool = True, ulysses: bool = True) -> int:
    """Room for the activation gather / scatter slots and the largest weight gather / scatter slots, plus - when the
    mode uses them - ring attention's gathered K|V and dK|dV inboxes and the Ulysses receive buffers (two of each)."""
    d, i = cfg.hidden_size, cfg.intermediate_size
    act = n * tokens_per_rank * d * 2
    weights = (2 * i * d + d * i + cfg.vocab_size * d) * 2
    total = 2 * (2 * act) + 2 * (2 * weights) + (64 << 20)
    if ring:
        total += 4 * n * tokens_per_rank * 2 * cfg.num_key_value_heads * cfg.head_dim * 2
    if ulysses:
        total += 2 * (2 * (cfg.q_size + 2 * cfg.kv_size) + 2 * cfg.q_size) * tokens_per_rank * 2
    return total


def setup_fused_comm(ctx, cfg=None, tokens_per_rank: int = 0, data_bytes: int = 0, mode: Optional[str] = None) -> bool:
    """Create and register the symmetric heaps for ``ctx``'s groups.  Returns False (leaving the NCCL
    composition in place) when the world is a single rank, the device is not CUDA, or peer memory
    cannot be set up."""
    from ..ops import fused_comm, native
    if ctx.world_size == 1 or ctx.device.type != "cuda" or not native.available():
        return False
    groups = []
    for g in (ctx.inner_group, ctx.world_group, ctx.ring_group):
        if g is not None and dist.get_world_size(g) > 1 and all(g is not h for h in groups):
            groups.append(g)
    ok = False
    for g in groups:
        if fused_comm.heap_for(g) is not None:
            ok = True
            continue
        # ``mode`` (when given) leaves out what that mode never allocates: K|V slots without a ring, receive buffers
        # outside Ulysses.  (A ring block holds inner_size x more tokens but 1 / inner_size of the heads: same bytes.)
        want_ring = ctx.ring_size > 1 or mode is None
        want_ulysses = mode in (None, "ulysses") and ctx.inner_size > 1
        nbytes = data_bytes or (heap_bytes_estimate(cfg, tokens_per_rank, dist.get_world_size(g), want_ring, want_ulysses)
                                if cfg is not None else (1 << 30))
        try:
            heap = SymmetricHeap(g, ctx.device, nbytes)
        except Exception as e:  # noqa: BLE001
            if ctx.rank == 0:
                print(f"[odysseus_transformer_b200] symmetric memory unavailable ({type(e).__name__}: {e}); using NCCL collectives")
            return False
        fused_comm.register_heap(g, heap)
        ok = True
    ctx.symm = ok
    if ok and ctx.wait_acc is None:
        # the fused kernels add the time they spend waiting on other GPUs here (utils.metrics.exposed_comm_ms)
        ctx.wait_acc = torch.zeros(4, dtype=torch.int64, device=ctx.device)
        native.lib().set_wait_accumulator(ctx.wait_acc)
    return ok
