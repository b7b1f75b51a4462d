"""BASELINE config 1: tiny Llama on CPU/gloo; every parallel mode must reproduce the loss and every
parameter gradient of an independent single-process causal-SDPA model (rtol 1e-4)."""
import pytest
import torch

from dist_utils import run_distributed
from reference_model import reference_loss


def _ref(cfg_name, L, seed=0):
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.models.llama import random_hf_state_dict
    cfg = get_model_config(cfg_name)
    sd = random_hf_state_dict(cfg, seed)
    for v in sd.values():
        v.requires_grad_(True)
    g = torch.Generator().manual_seed(0)
    batch = torch.randint(cfg.vocab_size, (1, L + 1), generator=g)
    loss, _ = reference_loss(cfg, sd, batch[0, :-1], batch[0, 1:])
    loss.backward()
    return cfg, sd, batch, loss.detach()


def _run_mode(rank, world, mode, cfg_name, L, U, R):
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.parallel.apply import build_model, prepare_attn_inputs
    from odysseus_transformer_b200.utils.debug import export_hf_grads
    import torch.distributed as dist
    cfg, sd, batch, ref_loss = _ref(cfg_name, L)
    ctx = init_parallel_context(mode, U, R, device=torch.device("cpu"), backend="library")
    model = build_model(cfg, mode, ctx, dtype=torch.float32, seed=0)
    pos = torch.arange(L).unsqueeze(0)
    s = prepare_attn_inputs(mode, batch[:, :-1], pos, batch[:, 1:], rank, world, "cpu", U, R)
    gt = L * (world if mode == "dp" else 1)
    loss = model(s["local_input_ids"], s["local_position_ids"], labels=s["local_target_ids"], global_tokens=gt)
    loss.backward()
    total = loss.detach().clone()
    dist.all_reduce(total)
    grads = export_hf_grads(model)
    torch.testing.assert_close(total, ref_loss, rtol=1e-4, atol=1e-5)
    worst = 0.0
    for k, v in sd.items():
        torch.testing.assert_close(grads[k], v.grad, rtol=1e-4, atol=2e-6, msg=lambda m: f"{mode} grad {k}: {m}")
        worst = max(worst, (grads[k] - v.grad).abs().max().item())
    return float(total), worst


@pytest.mark.parametrize("mode", ["tpsp", "ulysses", "ring", "odysseus", "dp"])
def test_mode_matches_single_process_world2(mode):
    res = run_distributed(_run_mode, 2, mode, "tiny", 512, 0, 1)
    assert len(res) == 2


@pytest.mark.parametrize("mode", ["ulysses", "odysseus"])
def test_hybrid_2x2(mode):
    res = run_distributed(_run_mode, 4, mode, "tiny", 256, 2, 2)
    assert len(res) == 4


def test_gqa_world2_odysseus():
    run_distributed(_run_mode, 2, "odysseus", "tiny-gqa", 256, 0, 1)


def test_gqa_world2_ulysses_ring_hybrid():
    run_distributed(_run_mode, 4, "ulysses", "tiny-gqa", 256, 2, 2)


def test_single_process_matches_reference():
    from odysseus_transformer_b200.mesh import ParallelContext
    from odysseus_transformer_b200.parallel.apply import build_model
    from odysseus_transformer_b200.utils.debug import export_hf_grads
    cfg, sd, batch, ref_loss = _ref("tiny", 256)
    model = build_model(cfg, None, ParallelContext(), dtype=torch.float32, seed=0)
    pos = torch.arange(256).unsqueeze(0)
    loss = model(batch[:, :-1], pos, labels=batch[:, 1:])
    loss.backward()
    torch.testing.assert_close(loss.detach(), ref_loss, rtol=1e-5, atol=1e-6)
    grads = export_hf_grads(model)
    for k, v in sd.items():
        torch.testing.assert_close(grads[k], v.grad, rtol=1e-4, atol=2e-6)
