#!/usr/bin/env python
"""Fused compute+collective paths vs the NCCL + GEMM composition, on N GPUs of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29520 benchmarks/comm_bench.py --tokens 16384

Cases (Llama-2-7B shapes, bf16; ``tokens`` = global sequence length, sharded on sequence):
  ag_qkv     all-gather(x [L/N,4096]) -> GEMM with W [3*4096/N, 4096]
  oproj_rs   GEMM x [L,4096/N] W [4096,4096/N] -> reduce-scatter rows
  wag_gateup all-gather(W [2*11008/N,4096]) -> GEMM with x [L/N,4096]
  wag_dgrad  all-gather(W) along K -> dgrad GEMM
  wgrad_rs   wgrad GEMM dy^T x -> reduce-scatter of [2*11008, 4096]
  ulysses_block  one Ulysses attention block (QKV projection, exchanges, attention, output projection; ZeRO-3
             weights) forward + backward: exchanges inside the kernels vs separate NCCL all-to-alls
  ring_fwd   zigzag ring attention forward, 32 heads x 128, L/N tokens per rank (gemm_only = the same attention
  ring_bwd   launches on already-gathered K/V, no exchange); backward includes the fp32 dK/dV reduce-scatter

Each case is timed with CUDA events on the launching stream after warm-up, a 256 MB write between
iterations, and reduced as the max over ranks.  The roofline is the slower of FLOPs / measured bf16 peak
and bytes that must cross NVLink per GPU / 770 GB/s (the measured one-direction peer-copy rate).
Rank 0 prints one JSON line per case."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
NVLINK_GBS = 770.0


def peak_tflops():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["bf16_tflops"], "measured"
    return 1590.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--push-order", choices=["dest", "unit", "both"], default="dest")
    ap.add_argument("--cases", type=str, default="ag_qkv,oproj_rs,wag_gateup,wag_dgrad,wgrad_rs")
    a = ap.parse_args()
    from odysseus_transformer_b200.comm import symm, torch_backend as C
    from odysseus_transformer_b200.config import get_model_config
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.ops import functional as F, fused_comm, native
    native.set_backend("fused")
    ctx = init_parallel_context("odysseus", backend="fused")
    n, rank, dev, g = ctx.world_size, ctx.rank, ctx.device, ctx.world_group
    cfg = get_model_config("llama2-7b")
    assert symm.setup_fused_comm(ctx, cfg, a.tokens // n), "peer memory unavailable"
    heap = fused_comm.heap_for(g)
    d, i, L, t = 4096, 11008, a.tokens, a.tokens // n
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    tf, kind = peak_tflops()

    def rnd(*s):
        return torch.randn(*s, device=dev).mul_(0.1).to(torch.bfloat16)

    def timeit(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        v = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v.item())

    tag = ["dest"]

    def report(name, fused_ms, nccl_ms, gemm_ms, flops, link_bytes, shape):
        if rank != 0:
            return
        t_comp, t_link = flops / (tf * 1e9), link_bytes / (NVLINK_GBS * 1e6)
        roof = max(t_comp, t_link)
        print(json.dumps({"case": name, "push_order": tag[0], "n_gpus": n, "tokens": L, "shape": shape, "fused_ms": round(fused_ms, 4),
                          "nccl_plus_gemm_ms": round(nccl_ms, 4), "gemm_only_ms": round(gemm_ms, 4),
                          "speedup_vs_nccl": round(nccl_ms / fused_ms, 3), "roofline_ms": round(roof, 4),
                          "bound": "compute" if t_comp >= t_link else "link",
                          f"frac_of_roofline({kind} peak, 770 GB/s)": round(roof / fused_ms, 3)}), flush=True)

    def timeline(name, fn):
        """Exposed communication of one gather launch: how long producers waited for rows, and the push span."""
        st = heap.enable_stats()
        fn()
        torch.cuda.synchronize()
        v = st.view(-1, 4).cpu()
        v = v[v[:, 3] > 0]
        t0 = int(v[:, 0][v[:, 0] > 0].min())
        if rank == 0:
            print(json.dumps({"case": name + "_timeline", "ctas": int(v.shape[0]),
                              "push_span_us": round((int(v[:, 1].max()) - t0) / 1e3, 1),
                              "kernel_span_us": round((int(v[:, 3].max()) - t0) / 1e3, 1),
                              "producer_row_wait_us_mean": round(float(v[:, 2].float().mean()) / 1e3, 1),
                              "producer_row_wait_us_max": round(int(v[:, 2].max()) / 1e3, 1)}), flush=True)
        heap.stats = None

    cases = a.cases.split(",")
    orders = ["dest", "unit"] if a.push_order == "both" else [a.push_order]
    for order in orders:
        # schedule of the comm warps: destination by destination (default) or every unit to all destinations at once
        native.lib().set_push_order(order == "unit")
        tag[0] = order
        if "ag_qkv" in cases:
            x, w = rnd(t, d), rnd(3 * d // n, d)
            fused = timeit(lambda: fused_comm._gather_gemm(heap, x, 1, w, 0))
            nccl = timeit(lambda: F.gemm_nt(C.all_gather_rows(x, g), w))
            xf = rnd(L, d)
            gemm = timeit(lambda: F.gemm_nt(xf, w))
            timeline("ag_qkv", lambda: fused_comm._gather_gemm(heap, x, 1, w, 0))
            report("ag_qkv", fused, nccl, gemm, 2.0 * L * d * (3 * d // n), (n - 1) * t * d * 2, [L, 3 * d // n, d])
        if "oproj_rs" in cases:
            x, w = rnd(L, d // n), rnd(d, d // n)
            fused = timeit(lambda: fused_comm._scatter_gemm(heap, x, w, 0, L, d))
            nccl = timeit(lambda: C.reduce_scatter_rows(F.gemm_nt(x, w), g))
            gemm = timeit(lambda: F.gemm_nt(x, w))
            report("oproj_rs", fused, nccl, gemm, 2.0 * L * d * (d // n), (n - 1) * t * d * 2, [L, d, d // n])
        if "wag_gateup" in cases:
            x, w = rnd(t, d), rnd(2 * i // n, d)
            fused = timeit(lambda: fused_comm._gather_gemm(heap, w, 2, x, 0))
            nccl = timeit(lambda: F.gemm_nt(x, C.all_gather_rows(w, g)))
            wf = rnd(2 * i, d)
            gemm = timeit(lambda: F.gemm_nt(x, wf))
            timeline("wag_gateup", lambda: fused_comm._gather_gemm(heap, w, 2, x, 0))
            report("wag_gateup", fused, nccl, gemm, 2.0 * t * d * 2 * i, (n - 1) * (2 * i // n) * d * 2, [t, 2 * i, d])
        if "wag_dgrad" in cases:
            dy, w = rnd(t, 2 * i), rnd(2 * i // n, d)
            fused = timeit(lambda: fused_comm._gather_gemm(heap, w, 2, dy, 1))
            nccl = timeit(lambda: F.gemm_nn(dy, C.all_gather_rows(w, g)))
            wf = rnd(2 * i, d)
            gemm = timeit(lambda: F.gemm_nn(dy, wf))
            timeline("wag_dgrad", lambda: fused_comm._gather_gemm(heap, w, 2, dy, 1))
            report("wag_dgrad", fused, nccl, gemm, 2.0 * t * d * 2 * i, (n - 1) * (2 * i // n) * d * 2, [t, d, 2 * i])
        if "wgrad_rs" in cases:
            dy, x = rnd(t, 2 * i), rnd(t, d)
            fused = timeit(lambda: fused_comm._scatter_gemm(heap, dy, x, 2, 2 * i, d))
            nccl = timeit(lambda: C.reduce_scatter_rows(F.gemm_tn(dy, x), g))
            gemm = timeit(lambda: F.gemm_tn(dy, x))
            report("wgrad_rs", fused, nccl, gemm, 2.0 * t * d * 2 * i, (n - 1) * (2 * i // n) * d * 2, [2 * i, d, t])
        if "ulysses_block" in cases:
            from odysseus_transformer_b200.ops import fused_ulysses
            from odysseus_transformer_b200.parallel.linear import Zero3Schedule
            from odysseus_transformer_b200.parallel.ulysses import SequenceParallelAttention
            sched = Zero3Schedule()
            blk = SequenceParallelAttention(cfg, ctx, sched, 0, dtype=torch.bfloat16, device=dev)
            for p_ in blk.parameters():
                torch.nn.init.normal_(p_, std=0.02)
            xb = rnd(t, d).requires_grad_(True)
            cos = torch.randn(L, 64, device=dev)
            sin = torch.randn(L, 64, device=dev)
            dyb = rnd(t, d)

            def step():
                for p_ in blk.parameters():
                    p_.grad = None
                xb.grad = None
                blk(xb, cos, sin).backward(dyb)

            assert fused_ulysses.available(blk, xb), "fused Ulysses block unavailable for this shape"
            fused = timeit(step)
            keep = fused_ulysses.available
            fused_ulysses.available = lambda *_: False
            nccl = timeit(step)
            fused_ulysses.available = keep
            # projections 4 * 2 t d^2 (fwd) * 3 (fwd + dgrad + wgrad), attention causal 3.5 * 4 L^2 hd H / 2 / n
            fl = 3 * 8.0 * t * d * d + 3.5 * 2.0 * L * L * 128 * 32 / n
            a2a_bytes = (n - 1) / n * t * (3 * d + d) * 2 * 2
            w_bytes = (n - 1) / n * 4 * d * d * 2 * 3
            report("ulysses_block", fused, nccl, 0.0, fl, a2a_bytes + w_bytes, [t, d, n])
        if "ring_fwd" in cases or "ring_bwd" in cases:
            from odysseus_transformer_b200.parallel import attention as PA
            H, hd = 32, 128
            sc = hd ** -0.5
            qkv = rnd(t, 3 * H, hd)
            q, k, v = qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]
            qc, kc, vc = q.contiguous(), k.contiguous(), v.contiguous()
            fake = rnd(n, 2, t, H, hd)
            lib, half = native.lib(), t // 2
            att_flops = 2.0 * L * L * hd * H / n             # causal: 4 L^2 hd H / 2, split over n ranks
            kv_bytes = (n - 1) * t * 2 * H * hd * 2

            def local_fwd():
                lib.attn_fwd(qc, kc, vc, True, sc)
                for s_ in range(1, n):
                    src = (rank - s_) % n
                    if src < rank:
                        lib.attn_fwd(qc, fake[src, 0, :half], fake[src, 1, :half], False, sc)
                    else:
                        lib.attn_fwd(qc[half:], fake[src, 0], fake[src, 1], False, sc)

            if "ring_fwd" in cases:
                fused = timeit(lambda: fused_comm.ring_attn_fwd(q, k, v, g, sc))
                nccl = timeit(lambda: PA.ring_attn_fwd(qc, kc, vc, g, sc))
                only = timeit(local_fwd)
                report("ring_fwd", fused, nccl, only, att_flops, kv_bytes, [t, H, hd])
            if "ring_bwd" in cases:
                o, lse = fused_comm.ring_attn_fwd(q, k, v, g, sc)
                do = rnd(t, H, hd)

                def local_bwd():
                    lib.attn_bwd(do, qc, kc, vc, o, lse, True, sc, None, None, None)
                    lse_hi = lse[:, half:].contiguous()
                    for s_ in range(1, n):
                        src = (rank - s_) % n
                        if src < rank:
                            lib.attn_bwd(do, qc, fake[src, 0, :half], fake[src, 1, :half], o, lse, False, sc, None, None, None)
                        else:
                            lib.attn_bwd(do[half:], qc[half:], fake[src, 0], fake[src, 1], o[half:], lse_hi, False, sc, None, None, None)

                fused = timeit(lambda: fused_comm.ring_attn_bwd(do, q, k, v, o, lse, g, sc))
                nccl = timeit(lambda: PA.ring_attn_bwd(do, qc, kc, vc, o, lse, g, sc))
                only = timeit(local_bwd)
                report("ring_bwd", fused, nccl, only, 2.5 * att_flops, 3 * kv_bytes, [t, H, hd])
    native.lib().set_push_order(False)
    native.check_status(dev.index)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
