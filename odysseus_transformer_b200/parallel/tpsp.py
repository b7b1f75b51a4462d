"""TP-SP (Megatron tensor parallel + sequence parallel) attention and MLP blocks.

``TPSPAttention`` is the attention block of both the ``tpsp`` and ``odysseus`` modes
(reference ``decoder/odysseus.py:45-271``): packed QKV projection as all-gather -> GEMM over the
inner group, RoPE on the gathered sequence, causal attention over the whole (ring-block) sequence
on ``H/U`` heads, output projection as GEMM -> reduce-scatter.  With a ring group of size R > 1 the
attention itself becomes zigzag ring attention across ring blocks (the Odysseus x ring hybrid the
reference README only claims, reference ``README.md:14``).

``TPSPMLP`` is the Megatron MLP (reference ``decoder/tensor_parallel.py:14-85``): packed
``w1w3`` column-parallel with a *local* ``[gate_u ; up_u]`` layout, ``w2`` row-parallel.
"""
from __future__ import annotations

from typing import Callable, Dict

import torch
import torch.nn as nn

from ..comm import torch_backend as C
from ..ops import functional as F
from .attention import packed_rope_attention
from .linear import ColumnParallelLinearAG, RowParallelLinearRS


class TPSPAttention(nn.Module):
    """``pack_weight=False`` keeps separate ``q_proj`` / ``k_proj`` / ``v_proj`` column-parallel linears (the
    reference's unpacked variant, reference ``decoder/odysseus.py:104-142``, which its attention test builds);
    the default packs them into one ``qkv_proj`` so the sequence is gathered once."""

    def __init__(self, cfg, ctx, layer_idx: int = 0, dtype=None, device=None, pack_weight: bool = True):
        super().__init__()
        U = ctx.inner_size
        self.cfg, self.pctx, self.layer_idx = cfg, ctx, layer_idx
        self.n_local_heads = cfg.num_attention_heads // U
        self.n_local_kv_heads = cfg.num_key_value_heads // U
        hd = cfg.head_dim
        self.head_dim = hd
        self.pack_weight = pack_weight
        if pack_weight:
            self.qkv_proj = ColumnParallelLinearAG(
                cfg.hidden_size, (self.n_local_heads + 2 * self.n_local_kv_heads) * hd, ctx.inner_group,
                dtype=dtype, device=device)
        else:
            mk = lambda heads: ColumnParallelLinearAG(cfg.hidden_size, heads * hd, ctx.inner_group,   # noqa: E731
                                                      dtype=dtype, device=device)
            self.q_proj, self.k_proj, self.v_proj = mk(self.n_local_heads), mk(self.n_local_kv_heads), mk(self.n_local_kv_heads)
        self.o_proj = RowParallelLinearRS(self.n_local_heads * hd, cfg.hidden_size, ctx.inner_group,
                                          dtype=dtype, device=device)
        if ctx.ring_size > 1:
            # replicated across ring blocks: their gradients are summed over the ring group
            for p in self.parameters():
                p.grad_sync_group = ctx.ring_group

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, residual=None) -> torch.Tensor:
        """x [T/N, d] local shard; cos/sin for the positions of this rank's ring block [T/R, hd/2].
        ``residual`` [T/N, d]: added to the block's output inside the output projection's kernel."""
        hq, hkv, hd = self.n_local_heads, self.n_local_kv_heads, self.head_dim
        rope = None
        if self.pack_weight:
            if F.epilogue_fusion("rope"):
                # q and k leave the projection rotated (GEMM epilogue); the attention op skips its own rotation
                rope = F.RopeEpilogue(cos, sin, (hq + hkv) * hd, (hq + 2 * hkv) * hd)
            qkv = self.qkv_proj(x, rope=rope)                    # [Tb, (hq + 2 hkv) * hd]
        else:
            qkv = torch.cat([self.q_proj(x), self.k_proj(x), self.v_proj(x)], dim=-1)
        o = packed_rope_attention(qkv, cos, sin, hq, hkv, self.pctx.ring_group,
                                  pre_rotated=rope is not None)  # [Tb, hq * hd]
        return self.o_proj(o, residual=residual)                 # [T/N, d]

    # -- HF state-dict <-> shard
    def hf_load(self, get: Callable[[str], torch.Tensor], prefix: str) -> None:
        u, hd = self.pctx.inner_rank, self.head_dim
        hq, hkv = self.n_local_heads, self.n_local_kv_heads
        wq = get(prefix + "q_proj.weight")[u * hq * hd:(u + 1) * hq * hd]
        wk = get(prefix + "k_proj.weight")[u * hkv * hd:(u + 1) * hkv * hd]
        wv = get(prefix + "v_proj.weight")[u * hkv * hd:(u + 1) * hkv * hd]
        with torch.no_grad():
            if self.pack_weight:
                self.qkv_proj.weight.copy_(torch.cat([wq, wk, wv], 0))
            else:
                self.q_proj.weight.copy_(wq)
                self.k_proj.weight.copy_(wk)
                self.v_proj.weight.copy_(wv)
            self.o_proj.weight.copy_(get(prefix + "o_proj.weight")[:, u * hq * hd:(u + 1) * hq * hd])

    def hf_export(self, prefix: str, out: Dict[str, torch.Tensor]) -> None:
        g, U, hd = self.pctx.inner_group, self.pctx.inner_size, self.head_dim
        hq, hkv = self.n_local_heads, self.n_local_kv_heads
        if not self.pack_weight:
            out[prefix + "q_proj.weight"] = self.q_proj.get_master_weight().clone()
            out[prefix + "k_proj.weight"] = self.k_proj.get_master_weight().clone()
            out[prefix + "v_proj.weight"] = self.v_proj.get_master_weight().clone()
            out[prefix + "o_proj.weight"] = self.o_proj.get_master_weight()
            return
        packed = C.all_gather_rows(self.qkv_proj.weight.detach(), g).view(U, (hq + 2 * hkv) * hd, -1)
        out[prefix + "q_proj.weight"] = packed[:, :hq * hd].reshape(U * hq * hd, -1).clone()
        out[prefix + "k_proj.weight"] = packed[:, hq * hd:(hq + hkv) * hd].reshape(U * hkv * hd, -1).clone()
        out[prefix + "v_proj.weight"] = packed[:, (hq + hkv) * hd:].reshape(U * hkv * hd, -1).clone()
        out[prefix + "o_proj.weight"] = self.o_proj.get_master_weight()


class TPSPMLP(nn.Module):
    def __init__(self, cfg, ctx, dtype=None, device=None):
        super().__init__()
        U = ctx.inner_size
        self.cfg, self.pctx = cfg, ctx
        self.i_local = cfg.intermediate_size // U
        self.w1w3 = ColumnParallelLinearAG(cfg.hidden_size, 2 * self.i_local, ctx.inner_group,
                                           dtype=dtype, device=device)
        self.w2 = RowParallelLinearRS(self.i_local, cfg.hidden_size, ctx.inner_group, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor, residual=None) -> torch.Tensor:
        return self.w2(F.swiglu(self.w1w3(x)), residual=residual)

    def hf_load(self, get, prefix: str) -> None:
        u, il = self.pctx.inner_rank, self.i_local
        with torch.no_grad():
            self.w1w3.weight.copy_(torch.cat([get(prefix + "gate_proj.weight")[u * il:(u + 1) * il],
                                              get(prefix + "up_proj.weight")[u * il:(u + 1) * il]], 0))
            self.w2.weight.copy_(get(prefix + "down_proj.weight")[:, u * il:(u + 1) * il])

    def hf_export(self, prefix: str, out) -> None:
        U, il = self.pctx.inner_size, self.i_local
        packed = C.all_gather_rows(self.w1w3.weight.detach(), self.pctx.inner_group).view(U, 2 * il, -1)
        out[prefix + "gate_proj.weight"] = packed[:, :il].reshape(U * il, -1).clone()
        out[prefix + "up_proj.weight"] = packed[:, il:].reshape(U * il, -1).clone()
        out[prefix + "down_proj.weight"] = self.w2.get_master_weight()
