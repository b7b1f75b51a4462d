"""Debug helpers: gradients in HF layout, poison fills.

``export_hf_grads`` returns every parameter's gradient as full HF-named tensors, using the same
gather logic as the checkpoint exporter, so gradients of any parallel mode can be compared with a
single-process model parameter by parameter (the reference's tests compare a few tensors pairwise
with loose tolerances, reference ``tests/mlp_test.py:81-88``).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..comm import torch_backend as C
from ..parallel.linear import wait_pending_grad_comm


def param_grad(p: torch.Tensor) -> torch.Tensor:
    if getattr(p, "main_grad", None) is not None and getattr(p, "_grad_written", False):
        return p.main_grad
    if p.grad is not None:
        return p.grad
    return torch.zeros_like(p)


def export_hf_grads(model) -> Dict[str, torch.Tensor]:
    wait_pending_grad_comm()
    params = list(model.parameters())
    stash = [p.data for p in params]
    try:
        for p in params:
            g = param_grad(p).detach().clone().to(p.dtype)
            grp = getattr(p, "grad_sync_group", None)
            if grp is not None:
                C.all_reduce_(g, grp)
            p.data = g
        return model.export_hf_state_dict()
    finally:
        for p, d in zip(params, stash):
            p.data = d


def poison_(t: torch.Tensor) -> torch.Tensor:
    """Fill a staging buffer with NaN so a read-before-arrival shows up in the result."""
    if t.is_floating_point():
        t.fill_(float("nan"))
    else:
        t.fill_(-1)
    return t
