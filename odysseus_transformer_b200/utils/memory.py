"""Per-GPU memory accounting of a training step: what is resident, what autograd keeps per layer, what fits.

The reference reports only measured peaks (``torch.cuda.max_memory_allocated`` printed by reference ``train.py:231-236``
and the OOM entries of its tables, reference ``README.md:39-45``); it has no way to say beforehand whether a sequence
length fits.  This module states the model the framework's own ops follow, term by term, so that a configuration can
be sized before it is launched (``python -m odysseus_transformer_b200.utils.memory --model llama2-7b --seq-length
131072 --gpus 8``) and so that the measured peaks can be checked against it.

Terms (bytes per GPU; N = world size, t = L / N local tokens, d hidden, I intermediate, q / kv = query / key-value
projection widths, V vocabulary; activations and weights are bf16):

* states: 16 bytes per locally owned parameter - bf16 working copy, bf16 flat gradient, fp32 master, two fp32 AdamW
  moments (``optim.adamw.ShardedAdamW``).  ZeRO-3 weights are owned 1/N each; the TP-SP attention weights 1/inner.
* saved activations per layer and local token (what the autograd functions of ``ops.functional`` keep): the two norm
  inputs and the two norm outputs (4 d), the rotated q|k|v (q + 2 kv), the attention output (q) with its fp32
  log-sum-exp (4 bytes per head), the gate|up pre-activation (2 I) and the SwiGLU output (I); the Ulysses block keeps
  the attention output twice, in head layout for the attention backward and in sequence layout for o_proj (q more).  Gathered weights and gathered sequences are
  never kept.
* with activation checkpointing only each layer's input (d) is kept, plus one layer's full set while it is recomputed.
* logits: t x V bf16, whose gradient is written in place (or ``loss_chunk_rows`` x V when the loss is chunked), plus the
  final norm's input and output (2 d per token).
* transients of backward: the gradients of one MLP (gate|up and SwiGLU output: 3 I per token), one packed dq|dk|dv
  (q + 2 kv) and the fp32 dQ accumulator of the attention backward (4 bytes x q per token, over the tokens the attention
  core sees).
* communication buffers: the symmetric heap (``comm.symm.heap_bytes_estimate``) on the fused backend, outside the
  caching allocator's statistics; on the library backend the two largest gathered weights.
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, Optional

GIB = float(1 << 30)


def _param_counts(cfg) -> Dict[str, int]:
    d, i = cfg.hidden_size, cfg.intermediate_size
    attn = d * (cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * d
    mlp = 3 * d * i
    return {"attn": attn * cfg.num_hidden_layers, "mlp": mlp * cfg.num_hidden_layers,
            "norms": (2 * cfg.num_hidden_layers + 1) * d, "tables": 2 * cfg.vocab_size * d}


def saved_bytes_per_token_per_layer(cfg, mode: str, inner: int = 1, fused: bool = True, elem: int = 2) -> int:
    """Bytes autograd keeps for one decoder layer and one local token (see the module docstring)."""
    d, i, q, kv = cfg.hidden_size, cfg.intermediate_size, cfg.q_size, cfg.kv_size
    elems = 4 * d + (q + 2 * kv) + q + 3 * i
    if mode == "ulysses" and inner > 1:
        elems += q                   # the attention output in head layout (attention) and in sequence layout (o_proj)
    stats = 4 * cfg.num_attention_heads + 2 * 4          # log-sum-exp per head, two rstd
    return elems * elem + stats


def estimate_memory(cfg, mode: str, seq_length: int, world: int, ulysses_degree: Optional[int] = None,
                    ring_degree: int = 1, grad_checkpoint: bool = False, loss_chunk_rows: int = 0,
                    use_zero3_linear: bool = True, fused: bool = True, elem: int = 2) -> Dict[str, float]:
    """Per-GPU estimate in GiB (the unit ``torch.cuda.max_memory_allocated`` is reported in by this package).

    ``peak_allocated`` is what the caching allocator should report; ``comm_heap`` comes on top of it in device
    memory on the fused backend."""
    if seq_length % world:
        raise ValueError(f"sequence length {seq_length} does not divide by {world} GPUs")
    inner = ulysses_degree if ulysses_degree else max(1, world // max(1, ring_degree))
    t = seq_length // world
    pc = _param_counts(cfg)
    if mode in ("odysseus", "tpsp"):
        owned = pc["attn"] / inner
        owned += pc["mlp"] / (world if (mode == "odysseus" and use_zero3_linear) else (1 if mode == "odysseus" else inner))
    else:
        owned = (pc["attn"] + pc["mlp"]) / world
    owned += pc["tables"] / world + pc["norms"]
    states = 16.0 * owned
    per_tok = saved_bytes_per_token_per_layer(cfg, mode, inner, fused, elem)
    layers = cfg.num_hidden_layers
    if grad_checkpoint:
        saved = layers * t * cfg.hidden_size * elem + t * per_tok
    else:
        saved = layers * t * per_tok
    rows = min(t, loss_chunk_rows) if loss_chunk_rows > 0 else t
    logits = rows * cfg.vocab_size * elem + 2 * t * cfg.hidden_size * elem
    t_attn = t * inner if mode in ("odysseus", "tpsp", "ulysses") else t     # tokens the attention core sees (heads / inner)
    transient = t * (3 * cfg.intermediate_size + cfg.q_size + 2 * cfg.kv_size) * elem + 4 * t_attn * cfg.q_size // inner
    comm = 0.0
    lib_buffers = 0.0
    if world > 1:
        if fused:
            from ..comm.symm import heap_bytes_estimate
            comm = float(heap_bytes_estimate(cfg, t, world, ring_degree > 1 or mode == "ring", mode == "ulysses"))
        else:
            lib_buffers = 2.0 * 2 * cfg.intermediate_size * cfg.hidden_size * elem
    if grad_checkpoint:
        # the logits are gone before the first layer is recomputed: the two do not add up
        kept = layers * t * cfg.hidden_size * elem
        peak = states + kept + max(logits, t * per_tok + transient) + lib_buffers
    else:
        peak = states + saved + logits + transient + lib_buffers
    out = {"states": states, "saved_activations": saved, "logits": logits, "backward_transients": transient,
           "library_gather_buffers": lib_buffers, "peak_allocated": peak, "comm_heap": comm, "total_device": peak + comm}
    return {k: v / GIB for k, v in out.items()}


def fits(est: Dict[str, float], device_gib: float = 178.0, headroom: float = 0.06) -> bool:
    """Whether the estimate leaves ``headroom`` of the device free (fragmentation, library workspaces, the context)."""
    return est["total_device"] <= device_gib * (1.0 - headroom)


def main(argv=None) -> int:
    from ..config import get_model_config
    ap = argparse.ArgumentParser(description="Per-GPU memory estimate of a training configuration")
    ap.add_argument("--model", default="llama2-7b")
    ap.add_argument("--mode", default="odysseus")
    ap.add_argument("--seq-length", type=int, default=65536)
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--ulysses-degree", type=int, default=0)
    ap.add_argument("--ring-degree", type=int, default=1)
    ap.add_argument("--grad-checkpoint", action="store_true")
    ap.add_argument("--loss-chunk-rows", type=int, default=0)
    ap.add_argument("--library", action="store_true", help="library backend (no symmetric heap)")
    a = ap.parse_args(argv)
    est = estimate_memory(get_model_config(a.model), a.mode, a.seq_length, a.gpus, a.ulysses_degree or None, a.ring_degree,
                          a.grad_checkpoint, a.loss_chunk_rows, fused=not a.library)
    est["fits_180GB"] = fits(est)
    print(json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in est.items()}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
