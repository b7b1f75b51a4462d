#!/usr/bin/env python
"""Single-kernel microbenchmarks on one GPU: own sm_100a kernels vs the library op, against the roofline.

    python benchmarks/kernel_bench.py gemm --m 8192 --n 12288 --k 4096 --layout 0
    python benchmarks/kernel_bench.py attn_fwd --t 8192 --heads 32
    python benchmarks/kernel_bench.py all            # the per-layer shapes of Llama-2-7B at 8K tokens

Timing: CUDA events on the launching stream, warm-up iterations first, and a 256 MB write between timed
iterations so nothing is served from the 126 MB L2.  Peaks come from MEASURED_PEAKS.json at the repository
root when present (copy bandwidth and cuBLAS bf16 rate measured on this pool), else the stated fallback.
Prints one JSON line per case."""
import argparse
import json
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def timeit(fn, iters=10, warmup=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def rnd(*shape):
    return torch.randn(*shape, device="cuda", dtype=torch.float32).mul_(0.5).to(torch.bfloat16)


def report(name, ms_own, ms_lib, flops=None, bytes_=None, **extra):
    hbm, tf, kind = peaks()
    rec = {"kernel": name, "ms": round(ms_own[0], 4), "ms_best": round(ms_own[1], 4)}
    if ms_lib is not None:
        rec["library_ms"] = round(ms_lib[0], 4)
        rec["speedup_vs_library"] = round(ms_lib[0] / ms_own[0], 3)
    if flops:
        rec["tflops"] = round(flops / ms_own[0] / 1e9, 1)
        rec[f"frac_of_{kind}_bf16_peak"] = round(flops / ms_own[0] / 1e9 / tf, 3)
    if bytes_:
        rec["gbs"] = round(bytes_ / ms_own[0] / 1e6, 1)
        rec[f"frac_of_{kind}_hbm"] = round(bytes_ / ms_own[0] / 1e6 / hbm, 3)
    rec.update(extra)
    print(json.dumps(rec), flush=True)


def bench_gemm(lib, M, N, K, layout, with_lib=True, iters=10):
    if layout == 0:
        a, b = rnd(M, K), rnd(N, K)
        ref = lambda: a @ b.t()
    elif layout == 1:
        a, b = rnd(M, K), rnd(K, N)
        ref = lambda: a @ b
    else:
        a, b = rnd(K, M), rnd(K, N)
        ref = lambda: a.t() @ b
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    own = timeit(lambda: lib.gemm(a, b, out, layout, False), iters)
    libt = timeit(ref, iters) if with_lib else None
    report(f"gemm_{['nt', 'nn', 'tn'][layout]}", own, libt, flops=2.0 * M * N * K, shape=[M, N, K])


def bench_attn(lib, T, H, Hkv, causal, which, with_lib=True, iters=10):
    from odysseus_transformer_b200.ops import functional as F
    q, k, v, do = rnd(T, H, 128), rnd(T, Hkv, 128), rnd(T, Hkv, 128), rnd(T, H, 128)
    scale = 1 / math.sqrt(128)
    o, lse = lib.attn_fwd(q, k, v, causal, scale)
    flops_fwd = 4.0 * T * T * H * 128 * (0.5 if causal else 1.0)
    if which == "fwd":
        own = timeit(lambda: lib.attn_fwd(q, k, v, causal, scale), iters)
        libt = timeit(lambda: F._aten_flash_fwd(q, k, v, causal, scale), iters) if with_lib else None
        report("attn_fwd", own, libt, flops=flops_fwd, shape=[T, H, Hkv], causal=causal)
    else:
        own = timeit(lambda: lib.attn_bwd(do, q, k, v, o, lse, causal, scale), iters)
        libt = timeit(lambda: F._aten_flash_bwd(do, q, k, v, o, lse, causal, scale), iters) if with_lib else None
        report("attn_bwd", own, libt, flops=2.5 * flops_fwd, shape=[T, H, Hkv], causal=causal)


def bench_elementwise(lib, T=8192, d=4096, I=11008, V=32000):
    from odysseus_transformer_b200.ops import torch_ref as R
    x, dl, w = rnd(T, d), rnd(T, d), rnd(d)
    own = timeit(lambda: lib.add_rmsnorm_fwd(x, dl, w, 1e-5))
    libt = timeit(lambda: R.add_rmsnorm_fwd(x, dl, w, 1e-5))
    report("add_rmsnorm_fwd", own, libt, bytes_=T * d * 2 * 4, shape=[T, d])
    y, rstd = lib.rmsnorm_fwd(x, w, 1e-5)
    own = timeit(lambda: lib.rmsnorm_bwd(dl, x, w, rstd, None))
    libt = timeit(lambda: R.rmsnorm_bwd(dl, x, w, rstd))
    report("rmsnorm_bwd", own, libt, bytes_=T * d * 2 * 3, shape=[T, d])
    gu, dh = rnd(T, 2 * I), rnd(T, I)
    own = timeit(lambda: lib.swiglu_fwd(gu))
    libt = timeit(lambda: R.swiglu_fwd(gu))
    report("swiglu_fwd", own, libt, bytes_=T * I * 2 * 3, shape=[T, I])
    own = timeit(lambda: lib.swiglu_bwd(dh, gu))
    libt = timeit(lambda: R.swiglu_bwd(dh, gu))
    report("swiglu_bwd", own, libt, bytes_=T * I * 2 * 5, shape=[T, I])
    logits = rnd(T, V)
    tg = torch.randint(0, V, (T,), device="cuda")
    own = timeit(lambda: lib.ce_fwd(logits, tg, -100))
    libt = timeit(lambda: R.cross_entropy_fwd(logits, tg, -100))
    report("ce_fwd", own, libt, bytes_=T * V * 2, shape=[T, V])
    n = 8 * 1024 * 1024 * 16
    master, m, v = torch.randn(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    g, p = rnd(n), torch.empty(n, device="cuda", dtype=torch.bfloat16)
    own = timeit(lambda: lib.adamw_step(master, m, v, g, p, 1e-4, 0.9, 0.999, 1e-8, 0.01, 2, 1.0))
    libt = timeit(lambda: R.adamw_step_(master, m, v, g, p, 1e-4, 0.9, 0.999, 1e-8, 0.01, 2, 1.0))
    report("adamw", own, libt, bytes_=n * 28, shape=[n])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "gemm_all", "attn_fwd", "attn_bwd", "elementwise", "all"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layout", type=int, default=0)
    ap.add_argument("--t", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--full", action="store_true", help="non-causal attention")
    ap.add_argument("--no-lib", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--gemm-variant", type=int, default=0, help="0 automatic, 1 one-CTA kernel, 2 CTA-pair kernel")
    ap.add_argument("--bwd-variant", type=int, default=1, help="attention backward: 0 fused dK/dV/dQ kernel, 1 split kernels")
    ap.add_argument("--fwd-kslice", type=int, default=-1, help="attention forward: 1 = Q / K tiles as 32-byte-swizzled slices, 0 = 128-byte halves")
    a = ap.parse_args()
    from odysseus_transformer_b200.ops import native
    native.set_backend("fused")
    lib = native.lib()
    lib.attn_bwd_set_variant(a.bwd_variant)
    if a.fwd_kslice >= 0:
        lib.attn_fwd_set_kslice(bool(a.fwd_kslice))
    lib.gemm_set_variant(a.gemm_variant)
    wl = not a.no_lib
    if a.what == "gemm":
        bench_gemm(lib, a.m, a.n, a.k, a.layout, wl, a.iters)
    elif a.what in ("attn_fwd", "attn_bwd"):
        bench_attn(lib, a.t, a.heads, a.kv_heads or a.heads, not a.full, a.what[5:], wl, a.iters)
    elif a.what == "elementwise":
        bench_elementwise(lib)
    else:
        T, d, I, V = 8192, 4096, 11008, 32000
        for (M, N, K, lay) in [(T, 3 * d, d, 0), (T, d, d, 0), (T, 2 * I, d, 0), (T, d, I, 0), (T, V, d, 0),
                               (T, d, 3 * d, 1), (T, d, 2 * I, 1), (T, I, d, 1),
                               (3 * d, d, T, 2), (2 * I, d, T, 2), (d, I, T, 2)]:
            bench_gemm(lib, M, N, K, lay, wl, a.iters)
        if a.what == "gemm_all":
            # the skinny 8-GPU shapes of the TP-SP attention linears: [65536, 1536, 4096] and K = 512
            for (M, N, K, lay) in [(65536, 1536, d, 0), (65536, d, 512, 0), (65536, d, 1536, 1), (1536, d, 65536, 2)]:
                bench_gemm(lib, M, N, K, lay, wl, a.iters)
            native.check_status(0)
            return
        bench_attn(lib, T, 32, 32, True, "fwd", wl, a.iters)
        bench_attn(lib, T, 32, 32, True, "bwd", wl, a.iters)
        bench_attn(lib, 32768, 4, 4, True, "fwd", wl, 5)
        bench_attn(lib, 32768, 4, 4, True, "bwd", wl, 5)
        bench_elementwise(lib)
    native.check_status(0)


if __name__ == "__main__":
    main()
