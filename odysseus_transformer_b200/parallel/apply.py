"""The parallel-mode switch: input sharding and model conversion.

Public surface kept from the reference:

* ``prepare_attn_inputs(parallel_mode, input_ids, position_ids, target_ids, rank, world_size, device)``
  (reference ``utils/apply_seq_parallel.py:132-144``) with the same result keys
  ``local_input_ids / local_position_ids / local_target_ids``;
* ``apply_odysseus_attn_patch_llama(model, use_zero3_linear)`` (reference ``decoder/odysseus.py:298``),
  ``apply_tpsp_attn_patch_llama(model)`` (reference ``decoder/tensor_parallel.py:88``),
  ``apply_ulysses_attn_monkey_patch_llama()`` (reference ``decoder/ulysses.py:109``),
  ``apply_zigzag_ring_attn_patch_llama()`` / ``..._mistral()`` (reference ``decoder/ring.py:99,108``).

Differences: the switch is one function, ``apply_seq_parallel(model, mode, ctx)``, which *re-shards the
weights the model already has* into the new mode (the reference re-initialises attention / MLP weights
and drops the loaded ones, reference ``decoder/odysseus.py:80-83``); nothing is patched globally; and
the input slicer also covers the inner x ring hybrid through two optional degree arguments.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config import PARALLEL_MODES, ModelConfig
from ..mesh import ParallelContext, block_indices, get_context, local_indices, mode_degrees


# ----------------------------------------------------------------------------- inputs


def extract_local(value: torch.Tensor, idx: torch.Tensor, device, dim: int = 1) -> torch.Tensor:
    return value.index_select(dim, idx.to(value.device)).to(device, non_blocking=True)


def extract_local_ulysses(value, rank, world_size, device, dim=1):
    """Contiguous shard ``[r*L/N, (r+1)*L/N)`` (reference ``extract_local_ulysses``)."""
    return extract_local(value, local_indices(value.shape[dim], world_size, 1, rank, 0), device, dim)


def extract_local_zigzag_ring(value, rank, world_size, device, dim=1):
    """Chunks ``r`` and ``2N-1-r`` of ``2N`` (reference ``extract_local_zigzag_ring``)."""
    return extract_local(value, local_indices(value.shape[dim], 1, world_size, 0, rank), device, dim)


def prepare_attn_inputs(parallel_mode: Optional[str], input_ids: torch.Tensor, position_ids: torch.Tensor,
                        target_ids: Optional[torch.Tensor], rank: int, world_size: int, device,
                        ulysses_degree: int = 0, ring_degree: int = 1) -> Dict[str, Optional[torch.Tensor]]:
    """Slice ``[1, L]`` ids / positions / targets for ``rank``.

    ulysses: contiguous shard of all three.  ring: zigzag shard of all three.  odysseus / tpsp:
    contiguous ids and targets but the positions of the *whole* attention span (RoPE runs after the
    sequence all-gather).  dp / None: everything.  With a hybrid (``ring_degree > 1``) the ring
    block is zigzag and the inner shard contiguous inside it; odysseus then gets its block's
    positions."""
    if parallel_mode not in PARALLEL_MODES and parallel_mode is not None:
        raise ValueError(f"Invalid parallel_mode: {parallel_mode}")
    if parallel_mode in (None, "dp"):
        return {"local_input_ids": input_ids.to(device), "local_position_ids": position_ids.to(device),
                "local_target_ids": None if target_ids is None else target_ids.to(device)}
    U, R = mode_degrees(parallel_mode, world_size, ulysses_degree, ring_degree)
    u, j = rank % U, rank // U
    L = input_ids.shape[1]
    idx = local_indices(L, U, R, u, j)
    out = {"local_input_ids": extract_local(input_ids, idx, device),
           "local_target_ids": None if target_ids is None else extract_local(target_ids, idx, device)}
    if parallel_mode in ("odysseus", "tpsp"):
        out["local_position_ids"] = extract_local(position_ids, block_indices(L, R, j), device)
    else:
        out["local_position_ids"] = extract_local(position_ids, idx, device)
    return out


# ----------------------------------------------------------------------------- model construction / conversion


def build_model(cfg: ModelConfig, mode: Optional[str], ctx: Optional[ParallelContext] = None,
                dtype: torch.dtype = torch.float32, device=None, seed: Optional[int] = 0,
                state_dict: Optional[Dict[str, torch.Tensor]] = None, use_zero3_linear: bool = True,
                loss_chunk_rows: int = 0):
    """Create the model directly in ``mode``; weights from ``state_dict`` (HF names) or random.
    ``use_zero3_linear=False`` (odysseus mode only) keeps the MLP weights whole on every rank."""
    from ..models.llama import LlamaForCausalLM
    ctx = ctx if ctx is not None else get_context()
    model = LlamaForCausalLM(cfg, mode, ctx, dtype=dtype, device=device, use_zero3_linear=use_zero3_linear,
                             loss_chunk_rows=loss_chunk_rows)
    if state_dict is not None:
        model.load_hf_state_dict(state_dict)
    elif seed is not None:
        model.init_weights(seed)
    return model


def apply_seq_parallel(model, mode: Optional[str], ctx: Optional[ParallelContext] = None,
                       use_zero3_linear: bool = True):
    """Return ``model`` converted to ``mode`` on mesh ``ctx``, keeping its weights.

    The weights are exported as a full HF state dict (gathering whatever sharding the model has
    now) and re-sharded into freshly built blocks of the new mode."""
    from ..models.llama import LlamaForCausalLM
    ctx = ctx if ctx is not None else get_context()
    sd = model.export_hf_state_dict()
    new = LlamaForCausalLM(model.cfg, mode, ctx, dtype=model.dtype_, device=model.embed_tokens.device,
                           use_zero3_linear=use_zero3_linear)
    new.load_hf_state_dict(sd)
    if getattr(model, "gradient_checkpointing", False):
        new.gradient_checkpointing_enable()
    return new


_DEFAULT_MODE: Optional[str] = None


def default_mode() -> Optional[str]:
    return _DEFAULT_MODE


def _apply(mode: str, model=None, use_zero3_linear: bool = True):
    global _DEFAULT_MODE
    if model is None:
        # the reference's argument-less patches change HF classes globally; the analogue here is a
        # process-wide default picked up by ``train`` / ``build_model`` callers that pass no mode
        _DEFAULT_MODE = mode
        return None
    return apply_seq_parallel(model, mode, use_zero3_linear=use_zero3_linear)


def apply_odysseus_attn_patch_llama(model=None, use_zero3_linear: bool = True):
    """TP-SP attention + sequence-parallel MLP (reference ``decoder/odysseus.py:298-309``).  With
    ``use_zero3_linear=False`` the MLP weights stay whole on every rank (``parallel.odysseus.ReplicatedMLP``)
    and their gradients are all-reduced once per step."""
    return _apply("odysseus", model, use_zero3_linear)


def apply_tpsp_attn_patch_llama(model=None):
    return _apply("tpsp", model)


def apply_ulysses_attn_monkey_patch_llama(model=None):
    return _apply("ulysses", model)


def apply_zigzag_ring_attn_patch_llama(model=None):
    return _apply("ring", model)


def apply_zigzag_ring_attn_patch_mistral(model=None):
    """Mistral shares the Llama block structure (no sliding window, as the reference asserts,
    decoder/ring.py:29); use the ``mistral-7b`` preset for its shapes."""
    return _apply("ring", model)
