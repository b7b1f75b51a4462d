"""Llama-family causal LM owned by this package.

The reference trains Hugging Face's ``LlamaForCausalLM`` and swaps or monkey-patches its attention
and MLP (reference ``train.py:66-100``).  This model keeps HF's *state-dict names and shapes* as
its checkpoint format but is built directly in the requested parallel mode:

====================  ==========================  ===========================
mode                  attention block             MLP block
====================  ==========================  ===========================
odysseus (+ring)      ``TPSPAttention``           ``OdysseusMLP`` (ZeRO-3), or
                                                  ``ReplicatedMLP`` with ``use_zero3_linear=False``
tpsp                  ``TPSPAttention``           ``TPSPMLP``
ulysses (+ring)       ``SequenceParallelAttention`` ``OdysseusMLP`` (ZeRO-3)
ring                  ``RingAttention``           ``OdysseusMLP`` (ZeRO-3)
dp / None             ``SequenceParallelAttention`` ``OdysseusMLP`` (ZeRO-3)
====================  ==========================  ===========================

Embedding and ``lm_head`` are vocab-sharded ZeRO-3 tables over the whole world; the norm weights
are replicated and their gradients all-reduced.  The loss is the **global mean** over all target
tokens of all ranks: every rank returns ``sum(local CE) / global_count`` so the partial losses add
up and every parameter receives exactly the gradient of that one scalar (the reference mixes
per-rank means with summed and averaged reductions, reference ``train.py:214-222``,
``utils/linear_zero3.py:82-84``).

Inter-layer activations are ``[T/N, d]``; the residual add happens in the epilogue of each block's output projection
(``ops.functional.fuse_epilogues``; otherwise it is fused into the following RMSNorm).
"""
from __future__ import annotations

import zlib
from typing import Callable, Dict, Optional

import torch
import torch.nn as nn

from ..comm import torch_backend as C
from ..config import ModelConfig
from ..mesh import ParallelContext, get_context
from ..ops import functional as F
from ..parallel.linear import LinearZeRO3, Zero3Schedule, zero3_embedding
from ..parallel.odysseus import OdysseusMLP, ReplicatedMLP
from ..parallel.ring import RingAttention
from ..parallel.tpsp import TPSPAttention, TPSPMLP
from ..parallel.ulysses import SequenceParallelAttention


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, ctx: ParallelContext, mode: Optional[str], layer_idx: int,
                 sched: Optional[Zero3Schedule], dtype, device, use_zero3_linear: bool = True, pack_qkv: bool = True):
        super().__init__()
        d = cfg.hidden_size
        self.eps = cfg.rms_norm_eps
        self.input_layernorm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        if mode in ("odysseus", "tpsp"):
            self.self_attn = TPSPAttention(cfg, ctx, layer_idx, dtype=dtype, device=device, pack_weight=pack_qkv)
        elif mode == "ring":
            self.self_attn = RingAttention(cfg, ctx, sched, layer_idx, dtype=dtype, device=device)
        else:
            self.self_attn = SequenceParallelAttention(cfg, ctx, sched, layer_idx, dtype=dtype, device=device)
        self.post_attention_layernorm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        if mode == "tpsp":
            self.mlp = TPSPMLP(cfg, ctx, dtype=dtype, device=device)
        elif mode == "odysseus" and not use_zero3_linear:
            self.mlp = ReplicatedMLP(cfg, ctx, dtype=dtype, device=device)
        else:
            self.mlp = OdysseusMLP(cfg, ctx, sched, dtype=dtype, device=device)
        for p in (self.input_layernorm, self.post_attention_layernorm):
            p.grad_sync_group = ctx.world_group

    def forward(self, x, delta, cos, sin):
        """(x, delta): residual stream and the not-yet-added output of the previous block (None when that block
        added it itself)."""
        if F.epilogue_fusion("residual"):
            # each block's output projection adds the residual stream in its own epilogue; the norms only normalise
            if delta is None:
                x, h = F.rmsnorm_keep(x, self.input_layernorm, self.eps)
            else:
                x, h = F.add_rmsnorm(x, delta, self.input_layernorm, self.eps)
            x = self.self_attn(h, cos, sin, residual=x)
            x, h = F.rmsnorm_keep(x, self.post_attention_layernorm, self.eps)
            return self.mlp(h, residual=x), None
        if delta is None:
            h = F.rmsnorm(x, self.input_layernorm, self.eps)
        else:
            x, h = F.add_rmsnorm(x, delta, self.input_layernorm, self.eps)
        a = self.self_attn(h, cos, sin)
        x, h = F.add_rmsnorm(x, a, self.post_attention_layernorm, self.eps)
        return x, self.mlp(h)


class LlamaForCausalLM(nn.Module):
    def __init__(self, cfg: ModelConfig, mode: Optional[str] = None, ctx: Optional[ParallelContext] = None,
                 dtype: torch.dtype = torch.float32, device=None, use_zero3_linear: bool = True,
                 loss_chunk_rows: int = 0, pack_qkv: bool = True):
        super().__init__()
        self.use_zero3_linear = use_zero3_linear
        # > 0: the training loss runs lm_head + cross-entropy this many tokens at a time (ops.functional.
        # linear_cross_entropy_sum) and lm_head stays out of the ZeRO-3 prefetch chain, whose order it would break
        self.loss_chunk_rows = int(loss_chunk_rows)
        if cfg.tie_word_embeddings:
            raise NotImplementedError("tied embeddings are not supported (Llama-2/3 do not tie)")
        ctx = ctx if ctx is not None else get_context()
        device = device if device is not None else ctx.device
        ctx.check_model(cfg, mode or "dp")
        self.cfg, self.mode, self.pctx = cfg, mode, ctx
        self.dtype_ = dtype
        n = C.group_size(ctx.world_group)
        if cfg.vocab_size % n:
            raise ValueError(f"vocab {cfg.vocab_size} must divide by world size {n} (ZeRO-3 tables)")
        self.zero3 = Zero3Schedule()
        self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size // n, cfg.hidden_size, dtype=dtype, device=device))
        self.layers = nn.ModuleList(
            [DecoderLayer(cfg, ctx, mode, i, self.zero3, dtype, device, use_zero3_linear, pack_qkv)
             for i in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
        self.norm.grad_sync_group = ctx.world_group
        self.lm_head = LinearZeRO3(cfg.hidden_size, cfg.vocab_size, ctx.world_group,
                                   None if self.loss_chunk_rows > 0 else self.zero3, dtype=dtype, device=device)
        self.gradient_checkpointing = False

    # ------------------------------------------------------------------ forward
    def rope_tables(self, position_ids: torch.Tensor):
        """cos/sin for the tokens the attention core sees on this rank (its whole ring block).

        ``position_ids`` follows ``prepare_attn_inputs``: the block's positions in odysseus / tpsp
        mode, the local tokens' positions otherwise (gathered over the inner group here)."""
        pos = position_ids.reshape(-1)
        if self.mode not in ("odysseus", "tpsp") and self.pctx.inner_size > 1:
            pos = C.all_gather_rows(pos.contiguous(), self.pctx.inner_group)
        return F.rope_tables(pos, self.cfg.head_dim, self.cfg.rope_theta)

    def hidden_states(self, input_ids: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
        ids = input_ids.reshape(-1)
        cos, sin = self.rope_tables(position_ids)
        if C.group_size(self.pctx.world_group) > 1:
            x = zero3_embedding(ids, self.embed_tokens, self.pctx.world_group)
        else:
            x = F.embedding(ids, self.embed_tokens)
        delta = None
        for layer in self.layers:
            if self.gradient_checkpointing and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                x, delta = checkpoint(layer, x, delta, cos, sin, use_reentrant=False)
            else:
                x, delta = layer(x, delta, cos, sin)
        if delta is None:
            return F.rmsnorm(x, self.norm, self.cfg.rms_norm_eps)
        _, h = F.add_rmsnorm(x, delta, self.norm, self.cfg.rms_norm_eps)
        return h

    def forward(self, input_ids: torch.Tensor, position_ids: torch.Tensor,
                labels: Optional[torch.Tensor] = None, global_tokens: Optional[int] = None):
        """Without ``labels``: logits ``[1, t, V]`` for the local tokens.  With ``labels`` (already
        shifted, local): this rank's share of the global-mean loss, ``sum(CE) / global_tokens``."""
        h = self.hidden_states(input_ids, position_ids)
        if labels is None:
            return self.lm_head(h).unsqueeze(0)                    # [1, t, V]
        tg = labels.reshape(-1)
        if global_tokens is None:
            global_tokens = tg.numel() * max(1, self.pctx.world_size)
        if self.loss_chunk_rows > 0:
            return F.linear_cross_entropy_sum(h, self.lm_head.weight, tg, 1.0 / float(global_tokens),
                                              self.lm_head.group, self.loss_chunk_rows)
        return F.cross_entropy_sum(self.lm_head(h), tg, 1.0 / float(global_tokens))

    def gradient_checkpointing_enable(self) -> None:
        """Recompute each decoder layer in backward (reference ``--grad-checkpoint``, train.py:161-162)."""
        self.gradient_checkpointing = True
        self.zero3.enabled = False

    # ------------------------------------------------------------------ HF state dict
    def hf_load(self, get: Callable[[str], torch.Tensor]) -> None:
        """Fill every shard from full HF-named tensors returned by ``get(name)``."""
        n = C.group_size(self.pctx.world_group)
        r = self.pctx.rank if n > 1 else 0
        vr = self.cfg.vocab_size // n
        with torch.no_grad():
            self.embed_tokens.copy_(get("model.embed_tokens.weight")[r * vr:(r + 1) * vr])
            self.lm_head.weight.copy_(get("lm_head.weight")[r * vr:(r + 1) * vr])
            self.norm.copy_(get("model.norm.weight"))
            for i, layer in enumerate(self.layers):
                p = f"model.layers.{i}."
                layer.input_layernorm.copy_(get(p + "input_layernorm.weight"))
                layer.post_attention_layernorm.copy_(get(p + "post_attention_layernorm.weight"))
                layer.self_attn.hf_load(get, p + "self_attn.")
                layer.mlp.hf_load(get, p + "mlp.")

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        dev, dt = self.embed_tokens.device, self.dtype_
        self.hf_load(lambda k: sd[k].to(device=dev, dtype=dt))

    def export_hf_state_dict(self) -> Dict[str, torch.Tensor]:
        """Gather every shard into full HF-named tensors (identical on all ranks)."""
        g = self.pctx.world_group
        out: Dict[str, torch.Tensor] = {}
        out["model.embed_tokens.weight"] = C.all_gather_rows(self.embed_tokens.detach(), g).clone()
        for i, layer in enumerate(self.layers):
            p = f"model.layers.{i}."
            out[p + "input_layernorm.weight"] = layer.input_layernorm.detach().clone()
            out[p + "post_attention_layernorm.weight"] = layer.post_attention_layernorm.detach().clone()
            layer.self_attn.hf_export(p + "self_attn.", out)
            layer.mlp.hf_export(p + "mlp.", out)
        out["model.norm.weight"] = self.norm.detach().clone()
        out["lm_head.weight"] = self.lm_head.get_master_weight().clone()
        return out

    def init_weights(self, seed: int = 0) -> None:
        """Random init N(0, initializer_range), identical for every mode and world size: each full
        HF tensor is generated from (seed, name) and sliced, so runs in different modes start from
        the same model."""
        self.hf_load(random_hf_tensors(self.cfg, seed, self.embed_tokens.device, self.dtype_))


def hf_param_shapes(cfg: ModelConfig) -> Dict[str, tuple]:
    d, i, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    shapes = {"model.embed_tokens.weight": (v, d), "model.norm.weight": (d,), "lm_head.weight": (v, d)}
    for n in range(cfg.num_hidden_layers):
        p = f"model.layers.{n}."
        shapes[p + "self_attn.q_proj.weight"] = (cfg.q_size, d)
        shapes[p + "self_attn.k_proj.weight"] = (cfg.kv_size, d)
        shapes[p + "self_attn.v_proj.weight"] = (cfg.kv_size, d)
        shapes[p + "self_attn.o_proj.weight"] = (d, cfg.q_size)
        shapes[p + "mlp.gate_proj.weight"] = (i, d)
        shapes[p + "mlp.up_proj.weight"] = (i, d)
        shapes[p + "mlp.down_proj.weight"] = (d, i)
        shapes[p + "input_layernorm.weight"] = (d,)
        shapes[p + "post_attention_layernorm.weight"] = (d,)
    return shapes


def random_hf_tensors(cfg: ModelConfig, seed: int, device, dtype) -> Callable[[str], torch.Tensor]:
    """``get(name)`` that synthesises the full HF tensor ``name`` deterministically on ``device``."""
    shapes = hf_param_shapes(cfg)
    device = torch.device(device)

    def get(name: str) -> torch.Tensor:
        shape = shapes[name]
        if name.endswith("layernorm.weight") or name == "model.norm.weight":
            return torch.ones(shape, dtype=dtype, device=device)
        g = torch.Generator(device=device)
        g.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFF)
        w = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * cfg.initializer_range
        return w.to(dtype)

    return get


def random_hf_state_dict(cfg: ModelConfig, seed: int = 0, device="cpu", dtype=torch.float32) -> Dict[str, torch.Tensor]:
    get = random_hf_tensors(cfg, seed, device, dtype)
    return {k: get(k) for k in hf_param_shapes(cfg)}
