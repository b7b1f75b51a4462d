"""Work folded into GEMM epilogues (rotary embedding in the q|k|v projection, residual in the output projections)
must not change the model: loss and every gradient with the fusions on equal those with them off, in every mode.
On CPU both settings run the library fallbacks of the same call sites the kernels serve on a GPU."""
import pytest
import torch

from dist_utils import run_distributed


def _loss_and_grads(rank, world, mode, rope, residual):
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.ops import functional as F
    from odysseus_transformer_b200.parallel.apply import build_model, prepare_attn_inputs
    F.fuse_epilogues(rope=rope, residual=residual)
    ctx = init_parallel_context(mode, device=torch.device("cpu"), backend="library")
    cfg = get_model_config("tiny")
    model = build_model(cfg, mode, ctx, dtype=torch.float32, seed=5)
    L = 64
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(cfg.vocab_size, (1, L), generator=g)
    pos = torch.arange(L).unsqueeze(0)
    labels = torch.roll(ids, -1, 1)
    s = prepare_attn_inputs(mode, ids, pos, labels, rank, world, "cpu")
    loss = model(s["local_input_ids"], s["local_position_ids"], s["local_target_ids"], global_tokens=L)
    loss.backward()
    grads = {n: p.grad.double().norm().item() for n, p in model.named_parameters() if p.grad is not None}
    return loss.item(), grads


@pytest.mark.parametrize("mode", ["odysseus", "tpsp", "ulysses", "ring"])
def test_fused_epilogues_leave_loss_and_gradients_unchanged(mode):
    off = run_distributed(_loss_and_grads, 2, mode, False, False)
    on = run_distributed(_loss_and_grads, 2, mode, True, True)
    for r in range(2):
        assert on[r][0] == pytest.approx(off[r][0], rel=1e-5, abs=1e-6)
        assert on[r][1].keys() == off[r][1].keys() and len(on[r][1]) > 0
        for name, v in off[r][1].items():
            assert on[r][1][name] == pytest.approx(v, rel=2e-4, abs=1e-7), name


def test_gemm_nt_epilogue_fallback_matches_separate_ops():
    from odysseus_transformer_b200.ops import functional as F, torch_ref as R
    T, hd, hq, hkv, groups = 12, 16, 4, 2, 2
    nh = hq + 2 * hkv
    a, b = torch.randn(T, 32), torch.randn(groups * nh * hd, 32)
    res = torch.randn(T, groups * nh * hd)
    cos, sin = R.rope_tables(torch.arange(T) * 3, hd, 10000.0)
    y = F.gemm_nt(a, b, rope=F.RopeEpilogue(cos, sin, (hq + hkv) * hd, nh * hd), residual=res)
    want = (a @ b.t()).view(T, groups, nh, hd).clone()
    for g in range(groups):
        want[:, g, :hq + hkv] = R.rope_apply(want[:, g, :hq + hkv], cos, sin)
    torch.testing.assert_close(y, want.view(T, -1) + res, rtol=1e-5, atol=1e-5)


def test_rmsnorm_keep_sums_both_gradients():
    from odysseus_transformer_b200.ops import functional as F
    x = torch.randn(9, 32, requires_grad=True)
    w = torch.randn(32, requires_grad=True)
    s, y = F.rmsnorm_keep(x, w, 1e-5)
    (s * 2.0).sum().add((y * y).sum()).backward()
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    y2 = F.rmsnorm(x2, w2, 1e-5)
    (x2 * 2.0).sum().add((y2 * y2).sum()).backward()
    torch.testing.assert_close(x.grad, x2.grad, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(w.grad, w2.grad, rtol=1e-5, atol=1e-6)
