"""Model and training configuration.

The reference takes its model hyper-parameters from a Hugging Face config object
(reference ``train.py:66-86``) and its run options from a flat argparse block
(reference ``train.py:243-263``).  Here both are plain dataclasses with named
presets so that synthetic, random-init runs need no network access.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Dict, Optional

PARALLEL_MODES = ("odysseus", "ulysses", "dp", "tpsp", "ring")


@dataclass
class ModelConfig:
    """Llama-family decoder hyper-parameters (field names follow HF ``LlamaConfig``)."""

    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_position_embeddings: int = 1 << 20
    initializer_range: float = 0.02
    tie_word_embeddings: bool = False
    name: str = "custom"

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def num_parameters(self) -> int:
        d, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        per_layer = d * self.q_size + 2 * d * self.kv_size + self.q_size * d + 3 * d * i + 2 * d
        return v * d * (1 if self.tie_word_embeddings else 2) + self.num_hidden_layers * per_layer + d

    def replace(self, **kw) -> "ModelConfig":
        return dataclasses.replace(self, **kw)

    def to_hf_dict(self) -> Dict:
        """Subset of an HF ``config.json`` that describes this architecture."""
        return {
            "architectures": ["LlamaForCausalLM"],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "initializer_range": self.initializer_range,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
        }

    @classmethod
    def from_hf_dict(cls, d: Dict) -> "ModelConfig":
        keys = {f.name for f in dataclasses.fields(cls)}
        kw = {k: v for k, v in d.items() if k in keys}
        if "num_key_value_heads" not in kw and "num_attention_heads" in kw:
            kw["num_key_value_heads"] = kw["num_attention_heads"]
        return cls(**kw)


def _presets() -> Dict[str, ModelConfig]:
    return {
        # 2-layer plumbing model used by the CPU/gloo parity tests.
        "tiny": ModelConfig(
            vocab_size=32000, hidden_size=256, intermediate_size=688, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=4, rms_norm_eps=1e-5, rope_theta=10000.0,
            name="tiny",
        ),
        # same, with grouped-query attention (2 KV heads)
        "tiny-gqa": ModelConfig(
            vocab_size=32000, hidden_size=256, intermediate_size=688, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5, rope_theta=10000.0,
            name="tiny-gqa",
        ),
        # head_dim 128 variant small enough for GPU unit tests of the sm_100a kernels
        "small": ModelConfig(
            vocab_size=32000, hidden_size=1024, intermediate_size=2816, num_hidden_layers=2,
            num_attention_heads=8, num_key_value_heads=8, name="small",
        ),
        "small-gqa": ModelConfig(
            vocab_size=32000, hidden_size=1024, intermediate_size=2816, num_hidden_layers=2,
            num_attention_heads=8, num_key_value_heads=2, name="small-gqa",
        ),
        "llama2-7b": ModelConfig(name="llama2-7b"),
        # the hard-coded "--use_cfg_init_model" model of the reference (train.py:66-76):
        # 16 layers, 32 query heads / 8 KV heads, otherwise Llama-2-7B shapes.
        "llama2-3b-gqa": ModelConfig(num_hidden_layers=16, num_key_value_heads=8, name="llama2-3b-gqa"),
        "llama3-8b": ModelConfig(
            vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
            num_attention_heads=32, num_key_value_heads=8, rope_theta=500000.0, name="llama3-8b",
        ),
        # Mistral-7B shapes without sliding window (the reference exposes a Mistral ring patch,
        # decoder/ring.py:108-114, and asserts the window off).
        "mistral-7b": ModelConfig(
            vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
            num_attention_heads=32, num_key_value_heads=8, rope_theta=10000.0, name="mistral-7b",
        ),
    }


MODEL_PRESETS = _presets()


def get_model_config(name: str, **overrides) -> ModelConfig:
    if name not in MODEL_PRESETS:
        raise KeyError(f"unknown model preset {name!r}; choose from {sorted(MODEL_PRESETS)}")
    cfg = MODEL_PRESETS[name]
    return cfg.replace(**overrides) if overrides else cfg


@dataclass
class TrainConfig:
    """Run options; the first block mirrors the reference CLI (train.py:243-263)."""

    batch_size: int = 1
    seed: int = 42
    max_train_steps: int = 10
    learning_rate: float = 2e-5
    rope_theta: Optional[float] = None
    model: str = "llama2-7b"
    seq_length: int = 16384
    cpu_offload: bool = False
    grad_checkpoint: bool = False
    use_zero2: bool = False
    use_ody_zero3: bool = True
    use_profiler: bool = False
    use_cfg_init_model: bool = False
    parallel_mode: Optional[str] = None
    # additions
    ulysses_degree: int = 0          # inner (Ulysses / Odysseus) degree of the hybrid; 0 = world size
    ring_degree: int = 1             # outer zigzag-ring degree of the hybrid
    backend: str = "auto"            # "fused" (sm_100a kernels) | "library" (NCCL + torch ops) | "auto"
    dtype: str = "bf16"
    weight_decay: float = 0.01
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    warmup_iterations: int = 2
    jsonl: Optional[str] = None
    save: Optional[str] = None
    load: Optional[str] = None
    data_on_device: bool = False
