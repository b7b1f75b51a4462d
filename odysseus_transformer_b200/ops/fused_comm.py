"""Single-kernel compute+collective paths over NVLink peer memory (sm_100a only).

``enabled(x, group)`` says whether the fused kernels serve this call: CUDA tensors, the ``fused``
backend, a multi-rank group and a symmetric heap registered for that group.  Otherwise callers run
the torch.distributed + GEMM composition in ``parallel.linear`` / ``parallel.attention``.
"""
from __future__ import annotations

from . import native

_heaps = {}   # id(group) -> comm.symm.SymmetricHeap


def register_heap(group, heap) -> None:
    _heaps[id(group)] = heap


def heap_for(group):
    return _heaps.get(id(group))


def enabled(x, group) -> bool:
    if group is None or not x.is_cuda or native.get_backend() == "library":
        return False
    return id(group) in _heaps and native.available()
