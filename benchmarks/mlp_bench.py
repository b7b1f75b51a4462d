#!/usr/bin/env python
"""Whole-MLP-block benchmark: the TP-SP MLP against the sequence-parallel ZeRO-3 (Odysseus) MLP, forward + backward.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29530 benchmarks/mlp_bench.py --tokens 65536

The reference times the same two blocks with ``benchmark_LlamaMLPTPSP`` and ``benchmark_LlamaMLPFSDP``
(reference ``tests/mlp_test.py:91-177``: ten forward + backward iterations on ``[1, seqlen, 4096]`` with
``i = 11008``, wall clock, the first without a device synchronisation).  Here each block runs on both backends -
``fused`` (own sm_100a GEMMs with the collective inside the kernel) and ``library`` (torch matmul + NCCL) - is timed
with CUDA events on the launching stream after warm-up with a 256 MB write between iterations, and reduced as the max
over ranks.  ``tokens`` is the global sequence length; every rank holds ``tokens / N`` of it.  Rank 0 prints one JSON
line per (block, backend): ms per forward + backward, model TFLOP/s per GPU, fraction of the measured bf16 peak, and
the activation / weight bytes the block moves per GPU (the reference's analysis: TP-SP moves activations,
``~ 4 L d`` elements per layer, Odysseus moves weights, ``~ 3 d i`` per direction; reference ``README.md:21-31``)."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def peak_tflops():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["bf16_tflops"], "measured"
    return 1590.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--model", type=str, default="llama2-7b")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--backends", type=str, default="fused,library")
    a = ap.parse_args()
    from odysseus_transformer_b200.comm import symm
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.ops import native
    from odysseus_transformer_b200.optim.adamw import ShardedAdamW
    from odysseus_transformer_b200.parallel.linear import Zero3Schedule, wait_pending_grad_comm
    from odysseus_transformer_b200.parallel.odysseus import OdysseusMLP
    from odysseus_transformer_b200.parallel.tpsp import TPSPMLP
    from odysseus_transformer_b200.utils.buffers import set_global_memory_buffer
    from odysseus_transformer_b200.utils.metrics import max_over_ranks

    ctx = init_parallel_context("tpsp", backend="fused")
    n, rank, dev = ctx.world_size, ctx.rank, ctx.device
    cfg = get_model_config(a.model)
    d, i, L = cfg.hidden_size, cfg.intermediate_size, a.tokens
    t = L // n
    set_global_memory_buffer(dev)
    native.set_backend("fused")
    if n > 1:
        assert symm.setup_fused_comm(ctx, cfg, t), "peer memory unavailable"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    tf, kind = peak_tflops()
    torch.manual_seed(rank)
    x = torch.randn(t, d, device=dev).mul_(0.5).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(t, d, device=dev).mul_(0.1).to(torch.bfloat16)

    def build(kind_):
        if kind_ == "tpsp":
            m = TPSPMLP(cfg, ctx, dtype=torch.bfloat16, device=dev)
        else:
            m = OdysseusMLP(cfg, ctx, Zero3Schedule(), dtype=torch.bfloat16, device=dev)
        for p in m.parameters():
            torch.nn.init.normal_(p, std=0.02)
        opt = ShardedAdamW(m.parameters(), lr=0.0)      # attaches main_grad: the wgrad GEMMs write there, as in training
        return m, opt

    def timeit(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            if n > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return max_over_ranks(ts[len(ts) // 2], dev)

    flops = 3 * 2 * 3 * L * d * i / n            # fwd + dgrad + wgrad of three [L, d] x [d, i] products, per GPU
    for block in ("tpsp", "odysseus"):
        m, opt = build(block)
        for backend in a.backends.split(","):
            native.set_backend(backend)

            def step():
                x.grad = None
                m(x).backward(dy)
                wait_pending_grad_comm()
                opt.zero_grad()

            ms = timeit(step)
            native.check_status(dev.index or 0)
            if rank == 0:
                act = (4 * L * d * 2 * (n - 1) / n) if block == "tpsp" else 0.0          # 2 AG + 2 RS of [L, d] fwd+bwd ... per GPU bytes in
                wts = 0.0 if block == "tpsp" else (2 * 3 * d * i * 2 * (n - 1) / n + 3 * d * i * 2 * (n - 1) / n)
                print(json.dumps({"block": block, "backend": backend, "n_gpus": n, "tokens": L, "ms_fwd_bwd": round(ms, 4),
                                  "tflops_per_gpu": round(flops / ms / 1e9, 1), "peak": kind,
                                  "frac_of_bf16_peak": round(flops / ms / 1e9 / tf, 3),
                                  "activation_bytes_in_per_gpu": act, "weight_bytes_in_per_gpu": wts}), flush=True)
        del m, opt
    native.set_backend("fused")
    if n > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
