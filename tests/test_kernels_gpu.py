"""sm_100a kernels against plain PyTorch fp32 references of the same op (needs a B200)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    from odysseus_transformer_b200.ops import native
    native.set_backend("fused")
    return native.lib()


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(dtype)


def _check_status(lib):
    torch.cuda.synchronize()
    assert lib.status(0) == 0, f"kernel status {lib.status(0)}"


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (384, 768, 320), (304, 264, 200), (1000, 72, 136),
               (2048, 4096, 1024), (8, 8, 8)]


@pytest.fixture(params=[1, 2], ids=["one_cta", "cta_pair"])
def gemm_variant(request, lib):
    """Run a GEMM test on the one-CTA kernel and on the cta_group::2 pair kernel; restore automatic choice after."""
    lib.gemm_set_variant(request.param)
    yield request.param
    lib.gemm_set_variant(0)


@pytest.mark.parametrize("layout", [0, 1, 2])
@pytest.mark.parametrize("M,N,K", GEMM_SHAPES + [(640, 1280, 192), (8192, 1536, 512)])
def test_gemm(lib, gemm_variant, layout, M, N, K):
    torch.manual_seed(M * 7 + N * 3 + K + layout)
    if layout == 0:
        a, b = _rand(M, K), _rand(N, K)
        ref = a.float() @ b.float().t()
    elif layout == 1:
        a, b = _rand(M, K), _rand(K, N)
        ref = a.float() @ b.float()
    else:
        a, b = _rand(K, M), _rand(K, N)
        ref = a.float().t() @ b.float()
    c = lib.gemm(a, b, None, layout, False)
    _check_status(lib)
    err = (c.float() - ref).abs().max().item()
    tol = 0.02 * math.sqrt(K) + 1e-2 * ref.abs().max().item()
    assert err <= tol, f"layout {layout} {M}x{N}x{K}: max err {err} > {tol}"
    # relative Frobenius error is the sharper check (catches a wrong k-slice or swizzle)
    rel = (c.float() - ref).norm() / ref.norm()
    assert rel < 5e-3, f"layout {layout} {M}x{N}x{K}: rel err {rel}"


@pytest.mark.parametrize("M", [300, 1024])
def test_gemm_rope_epilogue(lib, gemm_variant, M):
    """q|k|v projection whose epilogue rotates the q and k heads, against the fp32 product rotated in PyTorch."""
    from odysseus_transformer_b200.ops import torch_ref as R
    hq, hkv, hd, groups, K = 3, 1, 128, 2, 320
    nh = hq + 2 * hkv
    N = groups * nh * hd
    torch.manual_seed(M)
    a, b = _rand(M, K), _rand(N, K)
    pos = torch.randint(0, 100000, (M,), device="cuda")
    cos, sin = R.rope_tables(pos, hd, 10000.0)
    got = lib.gemm(a, b, None, 0, False, (cos, sin, (hq + hkv) * hd, nh * hd), None)
    _check_status(lib)
    want = (a.float() @ b.float().t()).view(M, groups, nh, hd).clone()
    for g in range(groups):
        want[:, g, :hq + hkv] = R.rope_apply(want[:, g, :hq + hkv], cos, sin, False)
    want = want.view(M, N)
    rel = (got.float() - want).norm() / want.norm()
    assert rel < 5e-3, rel
    # the v heads are the plain product, bit for bit
    plain = lib.gemm(a, b, None, 0, False)
    assert torch.equal(got.view(M, groups, nh, hd)[:, :, hq + hkv:], plain.view(M, groups, nh, hd)[:, :, hq + hkv:])
    assert not torch.equal(got.view(M, groups, nh, hd)[:, :, :hq], plain.view(M, groups, nh, hd)[:, :, :hq])
    # descriptions the kernel cannot take are refused before a launch
    with pytest.raises(RuntimeError):
        lib.gemm(a, b, None, 0, False, (cos[:-1], sin[:-1], (hq + hkv) * hd, nh * hd), None)      # a row short
    with pytest.raises(RuntimeError):
        lib.gemm(a, b, None, 0, False, (cos, sin, (hq + hkv) * hd, nh * hd + 64), None)          # period not whole heads
    with pytest.raises(RuntimeError):
        lib.gemm(a, b, None, 0, False, (cos.double(), sin.double(), (hq + hkv) * hd, nh * hd), None)
    with pytest.raises(RuntimeError):
        lib.gemm(a.t().contiguous(), b.t().contiguous(), None, 2, False, (cos, sin, (hq + hkv) * hd, nh * hd), None)


def test_gemm_residual_epilogue(lib, gemm_variant):
    M, N, K = 520, 640, 256
    a, b = _rand(M, K), _rand(N, K)
    wide = _rand(M, 2 * N)
    res = wide[:, N:]                          # strided residual rows
    out = lib.gemm(a, b, None, 0, False, None, res)
    _check_status(lib)
    ref = a.float() @ b.float().t() + res.float()
    assert ((out.float() - ref).norm() / ref.norm()) < 5e-3
    assert torch.equal(wide[:, N:], res)       # the residual itself is only read
    with pytest.raises(RuntimeError):
        lib.gemm(a, b, out, 0, True, None, res)                 # accumulate and residual exclude each other
    with pytest.raises(RuntimeError):
        lib.gemm(a, b, None, 0, False, None, res[:-1])          # wrong shape
    with pytest.raises(RuntimeError):
        lib.gemm(a, b, None, 0, False, None, res.float())       # wrong dtype


def test_gemm_accumulate_and_strided_out(lib, gemm_variant):
    M, N, K = 512, 384, 256
    a, b = _rand(K, M), _rand(K, N)
    base = _rand(M, N)
    out = base.clone()
    lib.gemm(a, b, out, 2, True)
    _check_status(lib)
    ref = base.float() + a.float().t() @ b.float()
    assert ((out.float() - ref).norm() / ref.norm()) < 5e-3
    # strided A (a column slice of a wider matrix) and strided out
    wide = _rand(M, 2 * K)
    w = _rand(N, K)
    big = torch.zeros(M, 2 * N, device="cuda", dtype=torch.bfloat16)
    lib.gemm(wide[:, K:], w, big[:, :N], 0, False)
    _check_status(lib)
    ref = wide[:, K:].float() @ w.float().t()
    assert ((big[:, :N].float() - ref).norm() / ref.norm()) < 5e-3
    assert big[:, N:].abs().max().item() == 0


@pytest.mark.parametrize("rows,dim", [(64, 256), (1000, 4096), (33, 1024), (17, 8192), (5, 16384), (601, 4096)])
def test_rmsnorm(lib, rows, dim):
    from odysseus_transformer_b200.ops import torch_ref as R
    x, d, w = _rand(rows, dim), _rand(rows, dim), _rand(dim) + 1
    y, rstd = lib.rmsnorm_fwd(x, w, 1e-5)
    yr, rr = R.rmsnorm_fwd(x, w, 1e-5)
    torch.testing.assert_close(y.float(), yr.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(rstd, rr, rtol=1e-4, atol=1e-5)
    s, y2, rstd2 = lib.add_rmsnorm_fwd(x, d, w, 1e-5)
    sr, y2r, r2r = R.add_rmsnorm_fwd(x, d, w, 1e-5)
    torch.testing.assert_close(s.float(), sr.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(y2.float(), y2r.float(), rtol=2e-2, atol=2e-2)
    dy, ds = _rand(rows, dim), _rand(rows, dim)
    dx, dw = lib.rmsnorm_bwd(dy, x, w, rstd, None)
    dxr, dwr = R.rmsnorm_bwd(dy, x, w, rr)
    torch.testing.assert_close(dx.float(), dxr.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dw, dwr, rtol=1e-3, atol=1e-2 * math.sqrt(rows))
    dx2, _ = lib.rmsnorm_bwd(dy, x, w, rstd, ds)
    torch.testing.assert_close(dx2.float(), dxr.float() + ds.float(), rtol=2e-2, atol=4e-2)


def test_rope(lib):
    from odysseus_transformer_b200.ops import torch_ref as R
    T, H, hd = 777, 6, 128
    pos = torch.randint(0, 200000, (T,), device="cuda")
    cos, sin = lib.rope_tables(pos, hd, 10000.0)
    cr, sr = R.rope_tables(pos, hd, 10000.0)
    torch.testing.assert_close(cos, cr, rtol=0, atol=2e-3)   # fp32 angles of ~2e5 rad carry ~1e-2 rad of rounding
    torch.testing.assert_close(sin, sr, rtol=0, atol=2e-3)
    x = _rand(T, H, hd)
    want = x.clone()
    want[:, :4] = R.rope_apply(x[:, :4], cr, sr, False)
    got = x.clone()
    lib.rope_inplace_(got, 4, cr, sr, False)
    torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-2)
    back = got.clone()
    lib.rope_inplace_(back, 4, cr, sr, True)
    torch.testing.assert_close(back.float(), x.float(), rtol=2e-2, atol=3e-2)
    # strided rows: rotate a slice of a wider packed tensor
    wide = _rand(T, 2 * H * hd)
    view = wide[:, :H * hd].view(T, H, hd) if False else wide.view(T, 2 * H, hd)
    ref = view.clone()
    ref[:, :3] = R.rope_apply(view[:, :3], cr, sr, False)
    lib.rope_inplace_(view, 3, cr, sr, False)
    torch.testing.assert_close(view.float(), ref.float(), rtol=1e-2, atol=1e-2)


def test_rope_grouped(lib):
    """Grouped rotation (first n_rot heads of every group of `period`), in place and as a copy, against fp32 PyTorch."""
    from odysseus_transformer_b200.ops import torch_ref as R
    T, groups, period, n_rot, hd = 389, 3, 5, 3, 128
    pos = torch.randint(0, 50000, (T,), device="cuda")
    cr, sr = R.rope_tables(pos, hd, 10000.0)
    x = _rand(T, groups * period, hd)
    want = x.float().view(T, groups, period, hd).clone()
    rot = R.rope_apply(x.view(T, groups, period, hd)[:, :, :n_rot].reshape(T, groups * n_rot, hd).float(), cr, sr, False)
    want[:, :, :n_rot] = rot.view(T, groups, n_rot, hd)
    want = want.view(T, groups * period, hd)
    out = torch.full_like(x, float("nan"))
    lib.rope_grouped_(x, out, n_rot, period, cr, sr, False)
    torch.testing.assert_close(out.float(), want, rtol=1e-2, atol=1e-2)
    # the heads that are not rotated are copied bit for bit
    assert torch.equal(out.view(T, groups, period, hd)[:, :, n_rot:], x.view(T, groups, period, hd)[:, :, n_rot:])
    inplace = x.clone()
    lib.rope_grouped_(inplace, inplace, n_rot, period, cr, sr, False)
    assert torch.equal(inplace, out)
    lib.rope_grouped_(inplace, inplace, n_rot, period, cr, sr, True)
    torch.testing.assert_close(inplace.float(), x.float(), rtol=2e-2, atol=3e-2)
    # strided source rows (a slice of a wider buffer) into a packed destination
    wide = _rand(T, 2 * groups * period * hd)
    src = wide[:, :groups * period * hd].unflatten(1, (groups * period, hd))
    out2 = torch.empty(T, groups * period, hd, device="cuda", dtype=torch.bfloat16)
    lib.rope_grouped_(src, out2, n_rot, period, cr, sr, False)
    ref2 = torch.empty_like(out2)
    lib.rope_grouped_(src.contiguous(), ref2, n_rot, period, cr, sr, False)
    assert torch.equal(out2, ref2)
    with pytest.raises(RuntimeError):
        lib.rope_grouped_(x, out, n_rot, 4, cr, sr, False)        # 15 heads are not groups of 4
    with pytest.raises(RuntimeError):
        lib.rope_grouped_(x, out[:, :5], n_rot, period, cr, sr, False)


def test_swiglu(lib):
    from odysseus_transformer_b200.ops import torch_ref as R
    T, I = 300, 2816
    gu, dh = _rand(T, 2 * I), _rand(T, I)
    torch.testing.assert_close(lib.swiglu_fwd(gu).float(), R.swiglu_fwd(gu).float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lib.swiglu_bwd(dh, gu).float(), R.swiglu_bwd(dh, gu).float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("T,V", [(64, 32000), (513, 128256), (7, 1000)])
def test_cross_entropy(lib, T, V):
    from odysseus_transformer_b200.ops import torch_ref as R
    logits = _rand(T, V, scale=3.0)
    tg = torch.randint(0, V, (T,), device="cuda")
    tg[::5] = -100
    loss, lse = lib.ce_fwd(logits, tg, -100)
    lr, lser = R.cross_entropy_fwd(logits, tg, -100)
    torch.testing.assert_close(lse, lser, rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(loss, lr, rtol=1e-4, atol=1e-3)
    scale = torch.tensor([1.0 / T], device="cuda")
    a, b = logits.clone(), logits.clone()
    lib.ce_bwd_(a, tg, lse, scale, -100)
    R.cross_entropy_bwd_(b, tg, lser, scale, -100)
    torch.testing.assert_close(a.float(), b.float(), rtol=2e-2, atol=1e-5)


def test_adamw(lib):
    from odysseus_transformer_b200.ops import torch_ref as R
    n = 8 * 100003
    master = torch.randn(n, device="cuda")
    m, v = torch.randn(n, device="cuda") * 0.01, torch.rand(n, device="cuda") * 1e-4
    g = _rand(n, scale=0.01)
    p = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    m2, v2, master2, p2 = m.clone(), v.clone(), master.clone(), p.clone()
    lib.adamw_step(master, m, v, g, p, 1e-3, 0.9, 0.999, 1e-8, 0.01, 3, 1.0)
    R.adamw_step_(master2, m2, v2, g, p2, 1e-3, 0.9, 0.999, 1e-8, 0.01, 3, 1.0)
    torch.testing.assert_close(master, master2, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(m, m2, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(v, v2, rtol=1e-5, atol=1e-9)
    torch.testing.assert_close(p.float(), p2.float(), rtol=1e-2, atol=1e-3)


def test_adamw_guard_word_blocks_the_update(lib):
    """A non-zero guard word (the step's kernel status) must leave master, moments and parameters untouched; zero lets it run."""
    n = 8 * 4099
    master, m, v = torch.randn(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    g = _rand(n, scale=0.01)
    p = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    keep = [t.clone() for t in (master, m, v, p)]
    guard = torch.tensor([105.0], device="cuda")
    lib.adamw_step(master, m, v, g, p, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1, 1.0, guard)
    for t, k in zip((master, m, v, p), keep):
        assert torch.equal(t, k)
    guard.zero_()
    lib.adamw_step(master, m, v, g, p, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1, 1.0, guard)
    assert not torch.equal(master, keep[0]) and not torch.equal(m, keep[1])
    with pytest.raises(RuntimeError):
        lib.adamw_step(master, m, v, g, p, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1, 1.0, torch.zeros(1))   # guard not on the device


def test_launchers_reject_mismatched_shapes_before_launching(lib):
    """Host-side checks only: every call below must raise without a kernel being launched (the launchers build tensor
    maps from the shapes they are told, so a mismatch would otherwise read past an allocation)."""
    lib.reset_launch_count()
    T, H = 256, 2
    q, k, v, o, do = (_rand(T, H, 128) for _ in range(5))
    lse = torch.zeros(H, T, device="cuda")
    bad = [
        lambda: lib.attn_bwd(do, q, k, _rand(T // 2, H, 128), o, lse, True, 0.1),          # v shorter than k
        lambda: lib.attn_bwd(do, q, k, _rand(T, 1, 128), o, lse, True, 0.1),               # v with fewer heads
        lambda: lib.attn_bwd(do, _rand(T, 3, 128), _rand(T, 2, 128), _rand(T, 2, 128), _rand(T, 3, 128),
                             torch.zeros(3, T, device="cuda"), True, 0.1),                   # 3 query heads on 2 kv heads
        lambda: lib.attn_bwd(do, q, k, v, o, torch.zeros(H, T), True, 0.1),                  # lse on the host
        lambda: lib.attn_bwd_split(do, q, k, _rand(T // 2, H, 128), o, lse, True, 0.1, [q], [k], [v]),
        lambda: lib.rmsnorm_bwd(_rand(8, 64), _rand(16, 64), _rand(64), torch.ones(16, device="cuda"), None),   # dy != x
        lambda: lib.rmsnorm_bwd(_rand(16, 64), _rand(16, 64), _rand(32), torch.ones(16, device="cuda"), None),  # short w
        lambda: lib.rmsnorm_bwd(_rand(16, 64), _rand(16, 64), _rand(64), torch.ones(8, device="cuda"), None),   # short rstd
        lambda: lib.rmsnorm_bwd(_rand(16, 64), _rand(16, 64), _rand(64), torch.ones(16), None),                 # rstd on host
        lambda: lib.rmsnorm_bwd(_rand(16, 64), _rand(16, 64), _rand(64), torch.ones(16, device="cuda"), _rand(8, 64)),
    ]
    for i, f in enumerate(bad):
        with pytest.raises(RuntimeError):
            f()
    assert lib.launch_count() == 0
    _check_status(lib)


def test_attn_merge(lib):
    from odysseus_transformer_b200.ops import torch_ref as R
    Tt, T, H, hd, row0 = 96, 48, 3, 128, 48
    out = torch.randn(Tt, H, hd, device="cuda")
    lse = torch.randn(H, Tt, device="cuda")
    o = _rand(T, H, hd)
    l = torch.randn(H, T, device="cuda")
    want_o, want_l = R.merge_attn(out[row0:], lse[:, row0:], o.float(), l)
    got_o, got_l = out.clone(), lse.clone()
    lib.attn_merge_(got_o, got_l, o, l, row0)
    torch.testing.assert_close(got_o[row0:], want_o, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(got_l[:, row0:], want_l, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(got_o[:row0], out[:row0])


def test_attn_merge_parts(lib):
    """One-pass merge of three partials, two of which cover only part of the rows."""
    T, H, hd = 96, 3, 128
    spans = [(0, 96), (0, 48), (48, 48)]
    os_ = [_rand(n, H, hd) for _, n in spans]
    ls_ = [torch.randn(H, n, device="cuda") for _, n in spans]
    got_o, got_l = lib.attn_merge_parts(os_, ls_, [b for b, _ in spans], T)
    lse = torch.full((H, T), float("-inf"), device="cuda")
    for (b, n), l in zip(spans, ls_):
        lse[:, b:b + n] = torch.logaddexp(lse[:, b:b + n], l)
    want = torch.zeros(T, H, hd, device="cuda")
    for (b, n), o, l in zip(spans, os_, ls_):
        want[b:b + n] += o.float() * torch.exp(l - lse[:, b:b + n]).t().unsqueeze(-1)
    torch.testing.assert_close(got_l, lse, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(got_o.float(), want, rtol=2e-2, atol=2e-2)


def test_sum_rows(lib):
    """Strided destination, sources landing on row sub-ranges, fp32 accumulation."""
    T, C = 80, 256
    big = _rand(T, C + 64)
    dst = big[:, 32:32 + C]
    srcs = [_rand(T, C), _rand(40, C), _rand(24, C + 8)[:, :C]]
    begins = [0, 0, 56]
    want = dst.float().clone()
    for sct, b in zip(srcs, begins):
        want[b:b + sct.shape[0]] += sct.float()
    keep = big.clone()
    lib.sum_rows_(dst, srcs, begins)
    torch.testing.assert_close(dst.float(), want, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(big[:, :32], keep[:, :32])
    torch.testing.assert_close(big[:, 32 + C:], keep[:, 32 + C:])


def test_model_step_fused_vs_library():
    """One fwd+bwd of the small model: own kernels vs the torch/cuBLAS/flash path, same weights."""
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.mesh import ParallelContext
    from odysseus_transformer_b200.ops import native
    from odysseus_transformer_b200.parallel.apply import build_model
    from odysseus_transformer_b200.utils.debug import export_hf_grads
    cfg = get_model_config("small")
    L = 512
    dev = torch.device("cuda", 0)
    ctx = ParallelContext(device=dev)
    g = torch.Generator().manual_seed(0)
    batch = torch.randint(cfg.vocab_size, (1, L + 1), generator=g).to(dev)
    pos = torch.arange(L, device=dev).unsqueeze(0)
    res = {}
    for be in ("library", "fused"):
        native.set_backend(be)
        model = build_model(cfg, "odysseus", ctx, dtype=torch.bfloat16, device=dev, seed=0)
        loss = model(batch[:, :-1], pos, labels=batch[:, 1:])
        loss.backward()
        res[be] = (loss.detach().float().item(), export_hf_grads(model))
    native.set_backend("fused")
    native.check_status(0)
    assert abs(res["fused"][0] - res["library"][0]) < 2e-2, (res["fused"][0], res["library"][0])
    for k, gl in res["library"][1].items():
        gf = res["fused"][1][k]
        denom = gl.float().norm().item() + 1e-6
        rel = (gf.float() - gl.float()).norm().item() / denom
        assert rel < 0.08, f"{k}: rel grad diff {rel}"


ATTN_CASES = [  # Tq, Tk, H, Hkv, causal
    (128, 128, 2, 2, True), (512, 512, 4, 2, True), (1000, 1000, 2, 1, True), (2048, 2048, 8, 8, True),
    (256, 384, 2, 2, False), (300, 200, 4, 1, False), (128, 1024, 2, 2, False),
    # the forward works on pairs of 128-row query tiles: an odd number of tiles, a ragged second tile, long loops
    (384, 384, 2, 2, True), (1408, 1408, 2, 1, True), (4096, 4096, 2, 2, True), (384, 520, 2, 2, False),
]


@pytest.fixture(params=[False, True], ids=["halves128", "slices32"])
def fwd_kslice(request, lib):
    """Both shared-memory layouts of the forward's Q / K tiles."""
    lib.attn_fwd_set_kslice(request.param)
    yield request.param
    lib.attn_fwd_set_kslice(False)


@pytest.mark.parametrize("Tq,Tk,H,Hkv,causal", ATTN_CASES)
def test_attention_fwd(lib, fwd_kslice, Tq, Tk, H, Hkv, causal):
    from odysseus_transformer_b200.ops import torch_ref as R
    torch.manual_seed(Tq + Tk + H)
    q, k, v = _rand(Tq, H, 128), _rand(Tk, Hkv, 128), _rand(Tk, Hkv, 128)
    scale = 1.0 / math.sqrt(128)
    o, lse = lib.attn_fwd(q, k, v, causal, scale)
    _check_status(lib)
    orf, lser = R.attn_fwd(q, k, v, causal, scale)
    torch.testing.assert_close(lse, lser, rtol=1e-3, atol=2e-3)
    torch.testing.assert_close(o.float(), orf.float(), rtol=2e-2, atol=2e-2)


def test_attention_fwd_growing_scores_rescale(lib):
    """Keys whose scores grow along the sequence move the running row maximum by more than 2^8 again and again,
    so the lazy rescaling of the output accumulator runs in (almost) every block."""
    from odysseus_transformer_b200.ops import torch_ref as R
    torch.manual_seed(5)
    T, H = 1024, 2
    q = _rand(T, H, 128).abs()
    ramp = torch.linspace(0.2, 6.0, T, device="cuda").view(T, 1, 1)
    k = (_rand(T, H, 128).abs().float() * ramp).to(torch.bfloat16)
    v = _rand(T, H, 128)
    scale = 1.0 / math.sqrt(128)
    for causal in (True, False):
        o, lse = lib.attn_fwd(q, k, v, causal, scale)
        _check_status(lib)
        orf, lser = R.attn_fwd(q, k, v, causal, scale)
        torch.testing.assert_close(o.float(), orf.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(lse, lser, rtol=1e-3, atol=2e-2)


def test_attention_fwd_packed_views(lib):
    """q/k/v as strided views of one packed [T, hq+2hkv, 128] tensor, peaked logits (rescale path)."""
    from odysseus_transformer_b200.ops import torch_ref as R
    T, hq, hkv = 640, 4, 2
    qkv = _rand(T, hq + 2 * hkv, 128, scale=3.0)
    q, k, v = qkv[:, :hq], qkv[:, hq:hq + hkv], qkv[:, hq + hkv:]
    scale = 1.0 / math.sqrt(128)
    o, lse = lib.attn_fwd(q, k, v, True, scale)
    _check_status(lib)
    orf, lser = R.attn_fwd(q, k, v, True, scale)
    torch.testing.assert_close(lse, lser, rtol=1e-3, atol=5e-3)
    torch.testing.assert_close(o.float(), orf.float(), rtol=3e-2, atol=3e-2)


@pytest.fixture(params=[0, 1], ids=["fused_dq", "split_dq"])
def bwd_variant(request, lib):
    """The fused dK/dV/dQ backward kernel and the split pair (dK/dV kernel + dQ kernel)."""
    lib.attn_bwd_set_variant(request.param)
    yield request.param
    lib.attn_bwd_set_variant(1)


@pytest.mark.parametrize("Tq,Tk,H,Hkv,causal", ATTN_CASES)
def test_attention_bwd(lib, bwd_variant, Tq, Tk, H, Hkv, causal):
    from odysseus_transformer_b200.ops import torch_ref as R
    torch.manual_seed(Tq * 3 + Tk + H)
    q, k, v = _rand(Tq, H, 128), _rand(Tk, Hkv, 128), _rand(Tk, Hkv, 128)
    do = _rand(Tq, H, 128)
    scale = 1.0 / math.sqrt(128)
    o, lse = R.attn_fwd(q, k, v, causal, scale)
    dq, dk, dv = lib.attn_bwd(do, q, k, v, o, lse, causal, scale)
    _check_status(lib)
    dqr, dkr, dvr = R.attn_bwd(do, q, k, v, o, lse, causal, scale)
    for name, a, b in (("dq", dq, dqr), ("dk", dk, dkr), ("dv", dv, dvr)):
        rel = ((a.float() - b).norm() / b.norm()).item()
        assert rel < 2e-2, f"{name}: rel err {rel}"
        torch.testing.assert_close(a.float(), b, rtol=5e-2, atol=5e-2 * b.abs().max().item(), msg=lambda m: f"{name}: {m}")


def test_attention_bwd_packed_outputs(lib, bwd_variant):
    """Gradients written straight into slices of one packed [T, hq+2hkv, 128] tensor."""
    from odysseus_transformer_b200.ops import torch_ref as R
    T, hq, hkv = 512, 4, 2
    qkv = _rand(T, hq + 2 * hkv, 128)
    q, k, v = qkv[:, :hq], qkv[:, hq:hq + hkv], qkv[:, hq + hkv:]
    do = _rand(T, hq, 128)
    scale = 1.0 / math.sqrt(128)
    o, lse = lib.attn_fwd(q, k, v, True, scale)
    dqkv = torch.full_like(qkv, float("nan"))
    lib.attn_bwd(do, q, k, v, o, lse, True, scale, dqkv[:, :hq], dqkv[:, hq:hq + hkv], dqkv[:, hq + hkv:])
    _check_status(lib)
    dqr, dkr, dvr = R.attn_bwd(do, q, k, v, o, lse, True, scale)
    ref = torch.cat([dqr, dkr, dvr], dim=1)
    assert torch.isfinite(dqkv.float()).all()
    assert ((dqkv.float() - ref).norm() / ref.norm()).item() < 2e-2
