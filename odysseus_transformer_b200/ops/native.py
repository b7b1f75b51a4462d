"""Loader for the in-tree sm_100a extension (``odysseus_transformer_b200/_C*.so``).

The reference has no native code of its own; every kernel it runs belongs to a dependency
(cuBLAS, flash-attn, Triton, NCCL).  Here the hot ops are hand-written CUDA in ``csrc/`` and are
built in-tree by ``build_ext.py``.  On a CUDA device with the ``fused`` backend selected a missing
extension is an error - there is no silent fallback to library kernels.
"""
from __future__ import annotations

import importlib
import os
import threading
from typing import Optional

_lock = threading.Lock()
_lib = None
_err: Optional[BaseException] = None
_backend = os.environ.get("ODY_BACKEND", "auto")  # "fused" | "library" | "auto"



def set_backend(name: str) -> None:
    """Select ``fused`` (own sm_100a kernels), ``library`` (torch / cuBLAS / NCCL), or ``auto``."""
    global _backend
    if name not in ("fused", "library", "auto"):
        raise ValueError(name)
    _backend = name


def get_backend() -> str:
    return _backend


def lib():
    """Import the extension (once). Raises if it is missing or fails to load."""
    global _lib, _err
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if _err is not None:
                raise RuntimeError(f"odysseus_transformer_b200._C failed to load earlier: {_err!r}")
            try:
                import torch  # noqa: F401  (libtorch symbols must be loaded first)
                _lib = importlib.import_module("odysseus_transformer_b200._C")
            except BaseException as e:  # noqa: BLE001
                _err = e
                raise RuntimeError(
                    "the sm_100a extension odysseus_transformer_b200._C is not built or failed to load; "
                    "run `python -m odysseus_transformer_b200.build_ext` (or __graft_entry__.build())"
                ) from e
    return _lib


def available() -> bool:
    try:
        lib()
        return True
    except RuntimeError:
        return False


def use_native(t) -> bool:
    """True when tensor ``t`` should go through the sm_100a kernels (CUDA, bf16 or integer)."""
    if not t.is_cuda or _backend == "library":
        return False
    if t.is_floating_point() and str(t.dtype) != "torch.bfloat16":
        return False
    if _backend == "fused":
        lib()          # raises loudly when the extension is missing
        return True
    return available()


def has_native_attention() -> bool:
    return available() and hasattr(lib(), "attn_fwd")


def has_native_attention_bwd() -> bool:
    return available() and hasattr(lib(), "attn_bwd")


def reset_launch_count() -> None:
    if available():
        lib().reset_launch_count()


def launch_count() -> int:
    """Launches of this package's own kernels since the last reset."""
    return int(lib().launch_count()) if available() else 0


class KernelStatusError(RuntimeError):
    """A bounded device-side wait gave up (codes in ``csrc/sm100.cuh``: 101-104 pipeline stages of one
    kernel, 105 a flag another GPU never set, 106 other)."""

    def __init__(self, status: int, where: str = ""):
        super().__init__(f"odysseus_transformer_b200 kernel reported status {status} "
                         f"(a bounded device-side wait expired){' ' + where if where else ''}")
        self.status = status


_status_source = None   # test hook: callable(device) -> 1-element tensor standing in for the device status word


def set_status_source(fn) -> None:
    """Replace the device status word by ``fn(device) -> tensor`` (``None`` restores the real one).
    Tests use it to exercise the failure branch of the training step without a failing kernel."""
    global _status_source
    _status_source = fn


def status_tensor(device):
    """The status word of ``device`` as a tensor on that device (first element), or ``None`` when there is
    none: no extension, or a CPU device without a test hook.  Reading it here costs no synchronisation, so a
    training step can fold it into a collective or hand it to the optimizer kernel as its guard."""
    if _status_source is not None:
        return _status_source(device)
    import torch
    device = torch.device(device)
    if device.type != "cuda" or _backend == "library" or not available():
        return None
    return lib().status_tensor(torch.empty(0, device=device))


def check_status(device_index: int = 0) -> None:
    """Raise if a bounded in-kernel wait gave up since the last check (codes in csrc/sm100.cuh)."""
    if not available():
        return
    st = int(lib().status(device_index))
    if st != 0:
        lib().clear_status(device_index)
        raise KernelStatusError(st)
