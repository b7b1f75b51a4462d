"""Odysseus blocks: TP-SP attention + sequence-parallel MLP with ZeRO-3 weights.

The MLP is the novelty of the reference (reference ``decoder/odysseus.py:274-295``,
``README.md:9-11``): tokens never leave their rank; the packed ``gate_up_proj`` ``[2i, d]`` (globally
``[gate ; up]``) and ``down_proj`` ``[d, i]`` are sharded on their first dim over the whole world,
gathered before each GEMM and their gradients reduce-scattered.  The attention block is
``parallel.tpsp.TPSPAttention``.  The same MLP serves the ulysses / ring / dp modes, where the
reference wraps an unsharded ``LlamaMLP`` in a single FSDP unit instead (reference
``train.py:115-126``).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import functional as F
from .linear import LinearZeRO3
from .tpsp import TPSPAttention  # noqa: F401  (re-exported: the attention half of the mode)


class OdysseusMLP(nn.Module):
    """``LlamaMLPZeRO`` of the reference."""

    def __init__(self, cfg, ctx, sched=None, dtype=None, device=None):
        super().__init__()
        self.cfg, self.pctx = cfg, ctx
        g = ctx.world_group
        self.gate_up_proj = LinearZeRO3(cfg.hidden_size, 2 * cfg.intermediate_size, g, sched, dtype=dtype, device=device)
        self.down_proj = LinearZeRO3(cfg.intermediate_size, cfg.hidden_size, g, sched, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(F.swiglu(self.gate_up_proj(x)))

    def hf_load(self, get, prefix: str) -> None:
        r, n = self.pctx.rank if self.pctx.world_group is not None else 0, max(1, self.pctx.world_size)
        gu = torch.cat([get(prefix + "gate_proj.weight"), get(prefix + "up_proj.weight")], 0)
        rows = gu.shape[0] // n
        dn = get(prefix + "down_proj.weight")
        drows = dn.shape[0] // n
        with torch.no_grad():
            self.gate_up_proj.weight.copy_(gu[r * rows:(r + 1) * rows])
            self.down_proj.weight.copy_(dn[r * drows:(r + 1) * drows])

    def hf_export(self, prefix: str, out) -> None:
        gu = self.gate_up_proj.get_master_weight()
        i = gu.shape[0] // 2
        out[prefix + "gate_proj.weight"] = gu[:i].clone()
        out[prefix + "up_proj.weight"] = gu[i:].clone()
        out[prefix + "down_proj.weight"] = self.down_proj.get_master_weight().clone()
