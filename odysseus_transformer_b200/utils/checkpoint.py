"""Checkpoint save / load in the Hugging Face Llama state-dict format, plus an optimizer sidecar.

The reference only *loads* (``AutoModelForCausalLM.from_pretrained``, reference ``train.py:78-86``)
and, in odysseus / tpsp mode, throws the loaded attention and MLP weights away when it swaps the
modules (reference ``decoder/odysseus.py:80-83``).  Here the interchange format is the unsharded HF
state dict (``model.layers.{n}.self_attn.q_proj.weight`` ...), written as ``pytorch_model.bin`` +
``config.json``; loading re-shards for whatever mode and world size the run uses, so a checkpoint
saved under one mode resumes under another.  Optimizer shards (fp32 master and moments), the step
and RNG state go to per-rank sidecar files, valid only for the same mode and world size.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..config import ModelConfig

WEIGHTS_NAME = "pytorch_model.bin"
CONFIG_NAME = "config.json"


def save_hf_checkpoint(model, path: str) -> None:
    """All ranks take part in the gather; rank 0 writes."""
    sd = model.export_hf_state_dict()
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        os.makedirs(path, exist_ok=True)
        torch.save({k: v.cpu() for k, v in sd.items()}, os.path.join(path, WEIGHTS_NAME))
        with open(os.path.join(path, CONFIG_NAME), "w") as f:
            json.dump(model.cfg.to_hf_dict(), f, indent=1)
    if dist.is_initialized():
        dist.barrier()


def load_hf_config(path: str) -> ModelConfig:
    with open(os.path.join(path, CONFIG_NAME)) as f:
        return ModelConfig.from_hf_dict(json.load(f))


def load_hf_state_dict_file(path: str) -> Dict[str, torch.Tensor]:
    """Read an HF checkpoint directory: ``pytorch_model.bin``, sharded ``*.bin`` with an index, or
    ``*.safetensors`` when the safetensors package is importable."""
    p = os.path.join(path, WEIGHTS_NAME)
    if os.path.exists(p):
        return torch.load(p, map_location="cpu", mmap=True, weights_only=True)
    idx = os.path.join(path, "pytorch_model.bin.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        sd: Dict[str, torch.Tensor] = {}
        for fn in files:
            sd.update(torch.load(os.path.join(path, fn), map_location="cpu", mmap=True, weights_only=True))
        return sd
    st = [f for f in os.listdir(path) if f.endswith(".safetensors")]
    if st:
        from safetensors.torch import load_file
        sd = {}
        for fn in sorted(st):
            sd.update(load_file(os.path.join(path, fn)))
        return sd
    raise FileNotFoundError(f"no HF weights found under {path}")


def load_hf_checkpoint(model, path: str) -> None:
    model.load_hf_state_dict(load_hf_state_dict_file(path))


def save_train_state(path: str, optimizer, step: int, rank: int, extra: Optional[dict] = None) -> None:
    os.makedirs(path, exist_ok=True)
    state = {"optimizer": {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in optimizer.state_dict().items()},
             "step": step, "torch_rng": torch.get_rng_state(), "extra": extra or {}}
    if torch.cuda.is_available():
        state["cuda_rng"] = torch.cuda.get_rng_state()
    torch.save(state, os.path.join(path, f"train_state_rank{rank}.pt"))


def load_train_state(path: str, optimizer, rank: int) -> int:
    state = torch.load(os.path.join(path, f"train_state_rank{rank}.pt"), map_location="cpu", weights_only=False)
    optimizer.load_state_dict(state["optimizer"])
    torch.set_rng_state(state["torch_rng"])
    if torch.cuda.is_available() and "cuda_rng" in state:
        torch.cuda.set_rng_state(state["cuda_rng"])
    return int(state["step"])
