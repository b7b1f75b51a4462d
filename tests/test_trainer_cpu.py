"""CPU tests of the training step: the kernel-status guard, optimizer offload, resume, and the optional modes
(ZeRO-2 style kept weights, activation checkpointing, the replicated-MLP Odysseus variant)."""
import os

import pytest
import torch

from dist_utils import run_distributed
from test_modes_cpu import _ref

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tiny_trainer(**kw):
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.mesh import ParallelContext
    from odysseus_transformer_b200.train import Trainer
    cfg = get_model_config("tiny")
    return cfg, Trainer(cfg, None, ParallelContext(), 64, lr=1e-2, dtype=torch.float32, seed=0, **kw)


def _batch(cfg, seed, L=64):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(cfg.vocab_size, (1, L + 1), generator=g)


# ----------------------------------------------------------------------------- status guard
def test_nonzero_kernel_status_skips_the_update_and_raises():
    """A status word that reads 105 (a peer flag never came) must (1) leave every weight and optimizer state as it
    was - decided by the optimizer's guard, not by the host - and (2) surface as KernelStatusError at the next call."""
    from odysseus_transformer_b200.ops import native
    cfg, tr = _tiny_trainer()
    word = torch.zeros(16, dtype=torch.int32)
    native.set_status_source(lambda device: word)
    try:
        tr.train_step(_batch(cfg, 0))                       # healthy step: weights move
        tr.check_status()
        before = tr.optimizer.master.clone()
        m_before = tr.optimizer.exp_avg.clone()
        word[0] = 105
        loss = tr.train_step(_batch(cfg, 1))                # the step itself returns; its update is a no-op
        assert torch.isfinite(loss)
        torch.testing.assert_close(tr.optimizer.master, before, rtol=0, atol=0)
        torch.testing.assert_close(tr.optimizer.exp_avg, m_before, rtol=0, atol=0)
        with pytest.raises(native.KernelStatusError) as ei:
            tr.train_step(_batch(cfg, 2))
        assert ei.value.status == 105 and "skipped" in str(ei.value)
        word[0] = 0
        tr.train_step(_batch(cfg, 3))                       # usable again once the status is clear
        tr.check_status()
        assert not torch.equal(tr.optimizer.master, before)
    finally:
        native.set_status_source(None)


def _status_two_ranks(rank, world):
    """One rank's status is non-zero: the all-reduced guard must stop the update on BOTH ranks."""
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.ops import native
    from odysseus_transformer_b200.train import Trainer
    cfg = get_model_config("tiny")
    ctx = init_parallel_context("odysseus", device=torch.device("cpu"), backend="library")
    tr = Trainer(cfg, "odysseus", ctx, 64, lr=1e-2, dtype=torch.float32, seed=0)
    word = torch.zeros(16, dtype=torch.int32)
    native.set_status_source(lambda device: word)
    try:
        tr.train_step(_batch(cfg, 0))
        before = tr.optimizer.master.clone()
        if rank == 1:
            word[0] = 105
        tr.train_step(_batch(cfg, 1))
        same = torch.equal(tr.optimizer.master, before)
        try:
            tr.check_status()
            raised = False
        except native.KernelStatusError:
            raised = True
        return same and raised
    finally:
        native.set_status_source(None)


def test_status_of_one_rank_stops_every_rank():
    res = run_distributed(_status_two_ranks, 2)
    assert res == {0: True, 1: True}


# ----------------------------------------------------------------------------- optimizer state on the host
def test_cpu_offload_optimizer_matches_resident_optimizer():
    from odysseus_transformer_b200.optim.adamw import ShardedAdamW
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(9, 8)), torch.nn.Parameter(torch.randn(16))]
    qs = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    a = ShardedAdamW(ps, lr=1e-2, weight_decay=0.1)
    b = ShardedAdamW(qs, lr=1e-2, weight_decay=0.1, cpu_offload=True)
    assert b.master.device.type == "cpu" and b.cpu_offload
    for _ in range(3):
        for p, q in zip(ps, qs):
            g = torch.randn_like(p)
            for t in (p, q):
                t.main_grad.copy_(g)
                t._grad_written = True
        a.step(); a.zero_grad()
        b.step(); b.zero_grad()
    for p, q in zip(ps, qs):
        torch.testing.assert_close(p.data, q.data, rtol=0, atol=0)
    # a raised guard leaves the offloaded state alone as well
    before = b.master.clone()
    for q in qs:
        q.main_grad.fill_(1.0)
        q._grad_written = True
    b.step(guard=torch.ones(1))
    torch.testing.assert_close(b.master, before, rtol=0, atol=0)


def test_train_cli_accepts_cpu_offload_and_replicated_mlp(tmp_path):
    from odysseus_transformer_b200.train import build_parser, main
    args = build_parser().parse_args(["--model-config", "tiny", "--seq-length", "64", "--max-train-steps", "3", "--dtype", "fp32",
                                      "--cpu-offload", "--parallel_mode", "odysseus", "--no_ody_zero3", "--backend", "library"])
    assert args.cpu_offload and not args.use_ody_zero3
    out = main(args)
    assert 9.0 < out["loss"] < 12.0


# ----------------------------------------------------------------------------- resume continues the data stream
def test_resume_continues_the_data_stream(tmp_path):
    """Steps 3 and 4 of a run resumed from a step-3 checkpoint must see the batches (hence the losses) that an
    uninterrupted 5-step run sees: the sidecar's RNG state is what the next batch is drawn from."""
    from odysseus_transformer_b200.train import build_parser, main
    common = ["--model-config", "tiny", "--seq-length", "64", "--dtype", "fp32", "--learning-rate", "1e-2", "--backend", "library"]
    full_log, part_log, res_log = (str(tmp_path / n) for n in ("full.jsonl", "part.jsonl", "res.jsonl"))
    main(build_parser().parse_args(common + ["--max-train-steps", "5", "--jsonl", full_log]))
    ck = str(tmp_path / "ck")
    main(build_parser().parse_args(common + ["--max-train-steps", "3", "--jsonl", part_log, "--save", ck]))
    main(build_parser().parse_args(common + ["--max-train-steps", "5", "--jsonl", res_log, "--load", ck]))
    import json
    def losses(path):
        return {r["step"]: r["loss"] for r in map(json.loads, open(path)) if "step" in r}
    full, res = losses(full_log), losses(res_log)
    assert sorted(res) == [3, 4]
    for s in (3, 4):
        assert abs(full[s] - res[s]) < 1e-5, (s, full[s], res[s])


# ----------------------------------------------------------------------------- optional modes against the single-process model
def _run_variant(rank, world, variant):
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.parallel.apply import build_model, prepare_attn_inputs
    from odysseus_transformer_b200.utils.debug import export_hf_grads
    import torch.distributed as dist
    L = 256
    cfg, sd, batch, ref_loss = _ref("tiny", L)
    mode = "ulysses" if variant == "zero2-ulysses" else "odysseus"
    ctx = init_parallel_context(mode, device=torch.device("cpu"), backend="library")
    model = build_model(cfg, mode, ctx, dtype=torch.float32, seed=0, use_zero3_linear=(variant != "replicated-mlp"),
                        loss_chunk_rows=48 if variant == "chunked-loss" else 0)     # 128 local tokens -> chunks of 48, 48, 32
    if variant.startswith("zero2"):
        model.zero3.keep_gathered = True
    if variant == "grad-checkpoint":
        model.gradient_checkpointing_enable()
    pos = torch.arange(L).unsqueeze(0)
    s = prepare_attn_inputs(mode, batch[:, :-1], pos, batch[:, 1:], rank, world, "cpu")
    worst = 0.0
    for it in range(2):           # twice: kept weights / recomputation must not leak state into the next step
        for p in model.parameters():
            p.grad = None
        loss = model(s["local_input_ids"], s["local_position_ids"], labels=s["local_target_ids"], global_tokens=L)
        loss.backward()
        total = loss.detach().clone()
        dist.all_reduce(total)
        torch.testing.assert_close(total, ref_loss, rtol=1e-4, atol=1e-5)
        grads = export_hf_grads(model)
        for k, v in sd.items():
            torch.testing.assert_close(grads[k], v.grad, rtol=1e-4, atol=2e-6, msg=lambda m: f"{variant} grad {k}: {m}")
            worst = max(worst, (grads[k] - v.grad).abs().max().item())
    if variant.startswith("zero2"):
        assert not model.zero3._kept, "kept weights must be released by backward"
    return type(model.layers[0].mlp).__name__


@pytest.mark.parametrize("variant", ["zero2", "zero2-ulysses", "grad-checkpoint", "replicated-mlp", "chunked-loss"])
def test_optional_modes_match_single_process_world2(variant):
    res = run_distributed(_run_variant, 2, variant)
    assert res[0] == ("ReplicatedMLP" if variant == "replicated-mlp" else "OdysseusMLP")


def _two_backwards(rank, world):
    """Two backward passes before one optimizer step: every gradient must be exactly twice the single one."""
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.optim.adamw import ShardedAdamW
    from odysseus_transformer_b200.parallel.apply import build_model, prepare_attn_inputs
    L = 128
    cfg, sd, batch, _ = _ref("tiny", L)
    ctx = init_parallel_context("odysseus", device=torch.device("cpu"), backend="library")
    model = build_model(cfg, "odysseus", ctx, dtype=torch.float32, seed=0)
    opt = ShardedAdamW(model.parameters(), lr=1e-3)
    pos = torch.arange(L).unsqueeze(0)
    s = prepare_attn_inputs("odysseus", batch[:, :-1], pos, batch[:, 1:], rank, world, "cpu")
    def bwd():
        model(s["local_input_ids"], s["local_position_ids"], labels=s["local_target_ids"], global_tokens=L).backward()
    bwd()
    opt.sync_grads()
    once = opt.flat_grad.clone()
    opt.zero_grad()
    bwd(); bwd()
    opt.sync_grads()
    torch.testing.assert_close(opt.flat_grad, 2 * once, rtol=1e-5, atol=1e-7)
    return True


def test_two_backwards_accumulate_world2():
    assert run_distributed(_two_backwards, 2) == {0: True, 1: True}


def test_default_loss_chunking_threshold():
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.train import default_loss_chunk_rows
    l2, l3 = get_model_config("llama2-7b"), get_model_config("llama3-8b")
    assert default_loss_chunk_rows(l2, 65536, 8, "odysseus", torch.bfloat16) == 0          # 8K tokens x 32000: 0.5 GB
    rows = default_loss_chunk_rows(l3, 262144, 8, "odysseus", torch.bfloat16)             # 32K tokens x 128256: 8.4 GB
    assert rows > 0 and rows % 128 == 0 and rows * l3.vocab_size * 2 <= (1 << 30)
