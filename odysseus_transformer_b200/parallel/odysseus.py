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

from ..comm import torch_backend as C
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

    def forward(self, x: torch.Tensor, residual=None) -> torch.Tensor:
        """``residual`` [T/N, d]: added to the block's output inside the down projection's kernel."""
        return self.down_proj(F.swiglu(self.gate_up_proj(x)), residual=residual)

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


class ReplicatedMLP(nn.Module):
    """Sequence-parallel MLP with whole weights on every rank: the ``use_zero3_linear=False`` variant of
    ``apply_odysseus_attn_patch_llama`` (reference ``decoder/odysseus.py:298-309``; its published
    "Odysseus (FSDP MLP)" rows, reference ``README.md:39-45``).

    Tokens stay local and no weight is gathered; the weight gradients of all ranks are summed by ONE
    all-reduce per step, issued by the optimizer over the flat gradient range of these parameters.  The
    reference leaves the plain ``LlamaMLP`` outside FSDP in this setting, so its gradients are never
    synchronised (reference ``train.py:128-132``); here they are.  Costs ``3 d i`` parameters plus their
    optimizer state per GPU instead of ``3 d i / N``."""

    def __init__(self, cfg, ctx, dtype=None, device=None):
        super().__init__()
        self.cfg, self.pctx = cfg, ctx
        d, i = cfg.hidden_size, cfg.intermediate_size
        self.gate_up_proj = nn.Parameter(torch.empty(2 * i, d, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(d, i, dtype=dtype, device=device))
        if ctx.world_group is not None and C.group_size(ctx.world_group) > 1:
            for p in self.parameters():
                p.grad_sync_group = ctx.world_group

    def forward(self, x: torch.Tensor, residual=None) -> torch.Tensor:
        y = F.linear(F.swiglu(F.linear(x, self.gate_up_proj)), self.down_proj)
        return y if residual is None else y + residual

    def hf_load(self, get, prefix: str) -> None:
        with torch.no_grad():
            self.gate_up_proj.copy_(torch.cat([get(prefix + "gate_proj.weight"), get(prefix + "up_proj.weight")], 0))
            self.down_proj.copy_(get(prefix + "down_proj.weight"))

    def hf_export(self, prefix: str, out) -> None:
        i = self.cfg.intermediate_size
        out[prefix + "gate_proj.weight"] = self.gate_up_proj.detach()[:i].clone()
        out[prefix + "up_proj.weight"] = self.gate_up_proj.detach()[i:].clone()
        out[prefix + "down_proj.weight"] = self.down_proj.detach().clone()
