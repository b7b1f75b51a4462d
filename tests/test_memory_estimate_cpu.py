"""The memory model of utils.memory: its saved-activation term against what autograd really keeps (saved-tensor hooks
on the CPU path, same autograd functions as on a GPU), and its totals against peaks measured on B200s."""
import pytest
import torch

from dist_utils import run_distributed


def _saved_bytes(rank, world, mode):
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.parallel.apply import build_model, prepare_attn_inputs
    from odysseus_transformer_b200.utils.memory import saved_bytes_per_token_per_layer
    ctx = init_parallel_context(mode, device=torch.device("cpu"), backend="library")
    cfg = get_model_config("tiny")
    model = build_model(cfg, mode, ctx, dtype=torch.float32, seed=5)
    L = 128
    ids = torch.randint(cfg.vocab_size, (1, L))
    s = prepare_attn_inputs(mode, ids, torch.arange(L).unsqueeze(0), torch.roll(ids, -1, 1), rank, world, "cpu")
    seen = {}

    def pack(t):
        seen.setdefault(t.untyped_storage().data_ptr(), (t.untyped_storage().nbytes(), tuple(t.shape)))
        return t

    with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        loss = model(s["local_input_ids"], s["local_position_ids"], s["local_target_ids"], global_tokens=L)
    params = {p.untyped_storage().data_ptr() for p in model.parameters()}
    t_local = L // world
    # per-layer tensors only: leave out parameters, the logits and what the final norm / lm_head keep
    per_layer = sum(nb for k, (nb, shp) in seen.items()
                    if k not in params and shp[-1] != cfg.vocab_size and nb >= t_local * 4 * 8)
    per_layer -= 2 * t_local * cfg.hidden_size * 4          # final norm input + lm_head input
    measured = per_layer / (t_local * cfg.num_hidden_layers)
    model_says = saved_bytes_per_token_per_layer(cfg, mode, inner=world, fused=False, elem=4)
    del loss
    return measured, model_says


@pytest.mark.parametrize("mode", ["odysseus", "tpsp", "ulysses", "ring"])
def test_saved_activation_model_matches_autograd(mode):
    res = run_distributed(_saved_bytes, 2, mode)
    for r in range(2):
        measured, model_says = res[r]
        # tables of cos / sin and a few per-token scalars are all that may differ
        assert measured == pytest.approx(model_says, rel=0.03), (mode, measured, model_says)


# (mode, L, GPUs, checkpointing, measured peak allocated GiB) on B200s, Llama-2-7B, fused backend
MEASURED = [("odysseus", 8192, 1, False, 133.2), ("odysseus", 32768, 4, False, 58.0), ("ulysses", 32768, 4, False, 60.0),
            ("ring", 32768, 4, False, 57.9), ("odysseus", 65536, 4, False, 90.8), ("ulysses", 65536, 4, False, 94.8),
            ("odysseus", 131072, 4, True, 38.55), ("odysseus", 131072, 8, False, 78.53), ("ulysses", 65536, 8, False, 47.66),
            ("tpsp", 65536, 8, False, 45.66), ("ring", 65536, 8, False, 45.64)]


@pytest.mark.parametrize("mode,L,n,ckpt,peak", MEASURED)
def test_estimate_matches_measured_peaks(mode, L, n, ckpt, peak):
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.utils.memory import estimate_memory
    est = estimate_memory(get_model_config("llama2-7b"), mode, L, n, grad_checkpoint=ckpt)
    assert est["peak_allocated"] == pytest.approx(peak, rel=0.06)


def test_what_fits():
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.utils.memory import estimate_memory, fits
    cfg = get_model_config("llama2-7b")
    assert fits(estimate_memory(cfg, "odysseus", 131072, 8))                        # 16K tokens per GPU
    assert not fits(estimate_memory(cfg, "odysseus", 262144, 4))                    # 64K tokens per GPU, no checkpointing
    assert fits(estimate_memory(cfg, "odysseus", 262144, 8, grad_checkpoint=True))
    with pytest.raises(ValueError):
        estimate_memory(cfg, "odysseus", 1000, 3)


def test_memory_cli_prints_one_json_line(capsys):
    import json
    from odysseus_transformer_b200.utils import memory
    assert memory.main(["--model", "llama2-7b", "--mode", "ulysses", "--seq-length", "65536", "--gpus", "8"]) == 0
    out = json.loads(capsys.readouterr().out.strip())
    assert out["fits_180GB"] is True and 40 < out["peak_allocated"] < 55
    assert memory.main(["--model", "llama2-7b", "--seq-length", "262144", "--gpus", "4"]) == 0
    assert json.loads(capsys.readouterr().out.strip())["fits_180GB"] is False
