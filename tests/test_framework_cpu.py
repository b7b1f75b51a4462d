"""CPU tests of the framework layer: input sharding, optimizer, checkpoint round trip, train CLI, buffers."""
import json
import os
import subprocess
import sys

import pytest
import torch

from dist_utils import run_distributed

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ----------------------------------------------------------------------------- input sharding
@pytest.mark.parametrize("mode,U,R", [("ulysses", 0, 1), ("ring", 0, 1), ("odysseus", 0, 1), ("tpsp", 0, 1),
                                      ("ulysses", 2, 2), ("odysseus", 2, 2), ("dp", 0, 1)])
def test_prepare_attn_inputs_partitions_the_sequence(mode, U, R):
    from odysseus_transformer_b200.parallel.apply import prepare_attn_inputs
    W, L = 4, 64
    ids = torch.arange(L).unsqueeze(0) + 1000
    pos = torch.arange(L).unsqueeze(0)
    tg = torch.arange(L).unsqueeze(0) + 2000
    seen = []
    for r in range(W):
        out = prepare_attn_inputs(mode, ids, pos, tg, r, W, "cpu", U, R)
        li, lp, lt = out["local_input_ids"], out["local_position_ids"], out["local_target_ids"]
        assert torch.equal(lt - 2000, li - 1000)
        if mode == "dp":
            assert li.shape[1] == L and torch.equal(lp, pos)
            continue
        assert li.shape[1] == L // W
        seen.append(li[0] - 1000)
        if mode in ("odysseus", "tpsp"):
            assert lp.shape[1] == L // max(1, R)              # positions of the whole attention span
            assert set((li[0] - 1000).tolist()) <= set(lp[0].tolist())
        else:
            assert torch.equal(lp[0], li[0] - 1000)
    if seen:
        assert sorted(torch.cat(seen).tolist()) == list(range(L))   # every token on exactly one rank


def test_zigzag_matches_reference_definition():
    from odysseus_transformer_b200.parallel.apply import extract_local_ulysses, extract_local_zigzag_ring
    v = torch.arange(32).unsqueeze(0)
    # rank r of 4 gets chunks r and 7-r of 8 (reference utils/apply_seq_parallel.py:93-98)
    assert extract_local_zigzag_ring(v, 1, 4, "cpu")[0].tolist() == [4, 5, 6, 7, 24, 25, 26, 27]
    assert extract_local_ulysses(v, 3, 4, "cpu")[0].tolist() == list(range(24, 32))


def test_mode_degrees_and_checks():
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.mesh import ParallelContext, mode_degrees
    assert mode_degrees("ring", 8) == (1, 8)
    assert mode_degrees("odysseus", 8, 4, 2) == (4, 2)
    assert mode_degrees("ulysses", 8) == (8, 1)
    with pytest.raises(ValueError):
        mode_degrees("tpsp", 8, 4, 2)
    with pytest.raises(ValueError):
        ParallelContext(world_size=8, inner_size=8).check_model(get_model_config("tiny"), "odysseus")   # 4 heads / 8


# ----------------------------------------------------------------------------- optimizer
def test_sharded_adamw_matches_torch_adamw_fp32():
    from odysseus_transformer_b200.optim.adamw import ShardedAdamW
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(13, 7)), torch.nn.Parameter(torch.randn(5))]
    qs = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    ref = torch.optim.AdamW(qs, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opt = ShardedAdamW(ps, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(4):
        gs = [torch.randn_like(p) for p in ps]
        for p, q, g in zip(ps, qs, gs):
            p.main_grad.copy_(g)
            p._grad_written = True
            q.grad = g.clone()
        opt.step()
        opt.zero_grad()
        ref.step()
    for p, q in zip(ps, qs):
        torch.testing.assert_close(p.data, q.data, rtol=1e-5, atol=1e-6)
    sd = opt.state_dict()
    opt2 = ShardedAdamW([torch.nn.Parameter(torch.zeros(13, 7)), torch.nn.Parameter(torch.zeros(5))], lr=1e-2)
    opt2.load_state_dict(sd)
    assert opt2.step_count == 4
    torch.testing.assert_close(opt2.params[0].data, ps[0].data)


def test_unwritten_and_autograd_grads_are_picked_up():
    from odysseus_transformer_b200.optim.adamw import ShardedAdamW
    p, q = torch.nn.Parameter(torch.ones(8)), torch.nn.Parameter(torch.ones(8))
    opt = ShardedAdamW([p, q], lr=0.1, weight_decay=0.0)
    (p * 2).sum().backward()                    # plain autograd gradient, q gets none
    before_q = q.detach().clone()
    opt.step()
    assert torch.all(p.detach() < 1.0)
    torch.testing.assert_close(q.detach(), before_q)


# ----------------------------------------------------------------------------- checkpoint round trip across modes
def _save_in_mode(rank, world, mode, path):
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.parallel.apply import build_model
    from odysseus_transformer_b200.utils import checkpoint as ckpt
    ctx = init_parallel_context(mode, device=torch.device("cpu"), backend="library")
    model = build_model(get_model_config("tiny"), mode, ctx, dtype=torch.float32, seed=3)
    ckpt.save_hf_checkpoint(model, path)
    return True


def _logits_in_mode(rank, world, mode, path):
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.parallel.apply import build_model, prepare_attn_inputs
    from odysseus_transformer_b200.utils import checkpoint as ckpt
    import torch.distributed as dist
    ctx = init_parallel_context(mode, device=torch.device("cpu"), backend="library")
    cfg = ckpt.load_hf_config(path)
    model = build_model(cfg, mode, ctx, dtype=torch.float32, seed=None, state_dict=ckpt.load_hf_state_dict_file(path))
    L = 64
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(cfg.vocab_size, (1, L), generator=g)
    pos = torch.arange(L).unsqueeze(0)
    s = prepare_attn_inputs(mode, ids, pos, None, rank, world, "cpu")
    with torch.no_grad():
        lg = model(s["local_input_ids"], s["local_position_ids"])[0]
    parts = [torch.empty_like(lg) for _ in range(world)]
    dist.all_gather(parts, lg)
    full = torch.cat(parts, 0)
    if mode == "ring":      # zigzag order -> natural order
        from odysseus_transformer_b200.mesh import local_indices
        idx = torch.cat([local_indices(L, 1, world, 0, r) for r in range(world)])
        full = full[torch.argsort(idx)]
    return full[:, :64].tolist()      # plain lists cross the process boundary without shared-memory handles


def test_checkpoint_saved_in_one_mode_loads_in_another(tmp_path):
    path = str(tmp_path / "ck")
    run_distributed(_save_in_mode, 2, "odysseus", path)
    assert os.path.exists(os.path.join(path, "pytorch_model.bin")) and os.path.exists(os.path.join(path, "config.json"))
    sd = torch.load(os.path.join(path, "pytorch_model.bin"), weights_only=True)
    assert sd["model.layers.1.self_attn.k_proj.weight"].shape == (256, 256)
    assert sd["model.layers.0.mlp.gate_proj.weight"].shape == (688, 256)
    a = torch.tensor(run_distributed(_logits_in_mode, 2, "ulysses", path)[0])
    b = torch.tensor(run_distributed(_logits_in_mode, 2, "ring", path)[0])
    c = torch.tensor(run_distributed(_logits_in_mode, 2, "tpsp", path)[0])
    torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(a, c, rtol=1e-4, atol=1e-5)


def _apply_switch(rank, world):
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.parallel.apply import apply_seq_parallel, apply_tpsp_attn_patch_llama, build_model
    ctx = init_parallel_context("odysseus", device=torch.device("cpu"), backend="library")
    m = build_model(get_model_config("tiny"), "odysseus", ctx, dtype=torch.float32, seed=5)
    sd0 = m.export_hf_state_dict()
    m2 = apply_seq_parallel(m, "ulysses", ctx)
    m3 = apply_tpsp_attn_patch_llama(m2)
    sd3 = m3.export_hf_state_dict()
    for k in sd0:
        torch.testing.assert_close(sd0[k], sd3[k])
    return type(m3.layers[0].mlp).__name__


def test_apply_seq_parallel_keeps_weights():
    res = run_distributed(_apply_switch, 2)
    assert res[0] == "TPSPMLP"


# ----------------------------------------------------------------------------- train CLI
def test_train_cli_two_ranks_gloo(tmp_path):
    out = tmp_path / "m.jsonl"
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(ROOT, "train.py"), "--parallel_mode", "odysseus", "--model-config", "tiny",
           "--seq-length", "128", "--max-train-steps", "5", "--dtype", "fp32", "--learning-rate", "1e-2",
           "--jsonl", str(out), "--save", str(tmp_path / "ck"), "--heartbeat-timeout", "30"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "odysseus 0K 2 Time taken:" in r.stdout
    assert "CUDA memory allocated" in r.stdout and "step 4, loss:" in r.stdout
    recs = [json.loads(l) for l in open(out)]
    losses = [x["loss"] for x in recs if "step" in x]
    # every step draws fresh random tokens (as the reference does), so the loss stays near ln(vocab)
    assert len(losses) == 5 and all(9.5 < l < 11.5 for l in losses)
    assert os.path.exists(tmp_path / "ck" / "train_state_rank1.pt")


def test_global_memory_buffer_reuses_storage():
    from odysseus_transformer_b200.utils.buffers import GlobalMemoryBuffer
    b = GlobalMemoryBuffer()
    t1 = b.get_tensor((4, 8), torch.float32, "mpu")
    t2 = b.get_tensor((2, 8), torch.float32, "mpu")
    assert t1.data_ptr() == t2.data_ptr()
    t3 = b.get_tensor((16, 8), torch.float32, "mpu")
    assert t3.numel() == 128 and b.bytes_held() == 128 * 4


def test_fused_paths_decline_on_cpu():
    """The fused compute+collective paths are CUDA-only: on CPU tensors every gate says no and the modules import."""
    import types

    import torch
    from odysseus_transformer_b200.comm import symm
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.ops import fused_comm, fused_ulysses

    x = torch.zeros(128, 8, 128, dtype=torch.bfloat16)
    assert not fused_comm.enabled(x, None)
    assert not fused_comm.ring_enabled(x, object())
    mod = types.SimpleNamespace(pctx=types.SimpleNamespace(inner_size=2, ring_size=1, inner_group=object(), world_group=object()),
                                head_dim=128)
    assert not fused_ulysses.available(mod, x)
    cfg = get_model_config("llama2-7b")
    small, big = symm.heap_bytes_estimate(cfg, 4096, 2), symm.heap_bytes_estimate(cfg, 8192, 8)
    assert 0 < small < big < 64 << 30
