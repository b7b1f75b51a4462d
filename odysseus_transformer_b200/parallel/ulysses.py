"""DeepSpeed-Ulysses attention block with ZeRO-3 weights (also the ring, hybrid and dp block).

The reference monkey-patches HF's attention to call ``yunchang.UlyssesAttention`` and leaves the
weights to one flat FSDP unit (reference ``decoder/ulysses.py:20-49,109-115``, ``train.py:115-126``).
Here the block owns its weights as ZeRO-3 shards over the whole world, projects QKV on the local
tokens, moves ``sequence <-> heads`` with ONE packed all-to-all over the inner group (q, k and v
travel together: the packed weight's rows are ordered by destination rank), runs the packed
RoPE + attention core over the ring group, and returns with one all-to-all before the output
projection.  Inner degree 1 gives pure zigzag ring attention (reference ``decoder/ring.py``); both
degrees 1 give plain local attention with ZeRO-3 weights (the ``dp`` mode).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..comm import torch_backend as C
from ..ops import functional as F
from .attention import head_to_seq, packed_rope_attention, seq_to_head
from .linear import LinearZeRO3


class SequenceParallelAttention(nn.Module):
    def __init__(self, cfg, ctx, sched=None, layer_idx: int = 0, dtype=None, device=None):
        super().__init__()
        self.cfg, self.pctx, self.layer_idx = cfg, ctx, layer_idx
        U = ctx.inner_size
        self.hq = cfg.num_attention_heads // U
        self.hkv = cfg.num_key_value_heads // U
        self.head_dim = cfg.head_dim
        g = ctx.world_group
        self.qkv_proj = LinearZeRO3(cfg.hidden_size, cfg.q_size + 2 * cfg.kv_size, g, sched, dtype=dtype, device=device)
        self.o_proj = LinearZeRO3(cfg.q_size, cfg.hidden_size, g, sched, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, residual=None) -> torch.Tensor:
        """x [t, d] local tokens; cos/sin for the positions of this rank's ring block [U*t, hd/2].
        ``residual`` [t, d]: added to the block's output inside the output projection's kernel."""
        U, hd = self.pctx.inner_size, self.head_dim
        t = x.shape[0]
        if U > 1 and x.is_cuda:
            from ..ops import fused_ulysses
            if fused_ulysses.available(self, x):
                # all four sequence<->head exchanges happen inside the GEMM / attention kernels
                return fused_ulysses.attention_block(self, x, cos, sin, residual)
        rope = None
        if F.epilogue_fusion("rope"):
            # q and k leave the projection rotated, at the positions of this rank's own tokens inside the block
            r = self.pctx.inner_rank if U > 1 else 0
            nh = self.hq + 2 * self.hkv
            rope = F.RopeEpilogue(cos[r * t:(r + 1) * t], sin[r * t:(r + 1) * t], (self.hq + self.hkv) * hd, nh * hd)
        qkv = self.qkv_proj(x, rope=rope)                                        # [t, U*(hq+2hkv)*hd]
        qkv = seq_to_head(qkv.view(t, U * (self.hq + 2 * self.hkv), hd), self.pctx.inner_group)
        o = packed_rope_attention(qkv.reshape(U * t, -1), cos, sin, self.hq, self.hkv, self.pctx.ring_group,
                                  pre_rotated=rope is not None)
        o = head_to_seq(o.view(U * t, self.hq, hd), self.pctx.inner_group)       # [t, H, hd]
        return self.o_proj(o.reshape(t, -1), residual=residual)

    def _packed_full(self, get, prefix):
        U, hd, hq, hkv = self.pctx.inner_size, self.head_dim, self.hq, self.hkv
        wq, wk, wv = get(prefix + "q_proj.weight"), get(prefix + "k_proj.weight"), get(prefix + "v_proj.weight")
        parts = []
        for u in range(U):
            parts += [wq[u * hq * hd:(u + 1) * hq * hd], wk[u * hkv * hd:(u + 1) * hkv * hd],
                      wv[u * hkv * hd:(u + 1) * hkv * hd]]
        return torch.cat(parts, 0)

    def hf_load(self, get, prefix: str) -> None:
        r = self.pctx.rank if self.pctx.world_group is not None else 0
        n = C.group_size(self.pctx.world_group)
        full = self._packed_full(get, prefix)
        rows = full.shape[0] // n
        wo = get(prefix + "o_proj.weight")
        orows = wo.shape[0] // n
        with torch.no_grad():
            self.qkv_proj.weight.copy_(full[r * rows:(r + 1) * rows])
            self.o_proj.weight.copy_(wo[r * orows:(r + 1) * orows])

    def hf_export(self, prefix: str, out) -> None:
        U, hd, hq, hkv = self.pctx.inner_size, self.head_dim, self.hq, self.hkv
        packed = self.qkv_proj.get_master_weight().view(U, (hq + 2 * hkv) * hd, -1)
        out[prefix + "q_proj.weight"] = packed[:, :hq * hd].reshape(U * hq * hd, -1).clone()
        out[prefix + "k_proj.weight"] = packed[:, hq * hd:(hq + hkv) * hd].reshape(U * hkv * hd, -1).clone()
        out[prefix + "v_proj.weight"] = packed[:, (hq + hkv) * hd:].reshape(U * hkv * hd, -1).clone()
        out[prefix + "o_proj.weight"] = self.o_proj.get_master_weight().clone()
