#!/usr/bin/env python
"""Run the fused gather / scatter GEMM on ONE GPU in loop-back form, for profilers that cannot follow a
multi-rank job (``ncu`` captures one process).

The kernel is launched as rank 0 of 2 with every "peer" pointer aimed at this GPU's own buffers: the comm
warps push rank 0's shard with the same st.global path they use across NVLink, the consumers gate their
TMA loads on the same arrival counters, and the counters that rank 1 would have raised are pre-set on the
host so nothing waits for a launch that does not exist.  Numbers from this script describe the kernel's
instruction mix and on-chip behaviour, not NVLink throughput (see benchmarks/comm_bench.py for that).

    python benchmarks/fused_loopback.py gather --tokens 8192       # all-gather(x) -> QKV GEMM
    python benchmarks/fused_loopback.py scatter --tokens 8192      # O-proj GEMM -> reduce-scatter
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gather", "scatter"])
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    from odysseus_transformer_b200.ops import native
    native.set_backend("fused")
    lib = native.lib()
    dev = torch.device("cuda", 0)
    n, d = 2, 4096
    L, t = a.tokens, a.tokens // n
    sms = torch.cuda.get_device_properties(dev).multi_processor_count

    def rnd(*s):
        return torch.randn(*s, device=dev).mul_(0.1).to(torch.bfloat16)

    if a.what == "gather":
        x, w = rnd(t, d), rnd(3 * d // n, d)
        gathered = rnd(L, d)                                  # rank 1's half already "arrived"
        nb = t // 128
        flags = torch.zeros(n * nb, dtype=torch.int32, device=dev)
        counters = torch.zeros(8, dtype=torch.int32, device=dev)
        free = torch.zeros(8, dtype=torch.int32, device=dev)
        done = torch.zeros(1, dtype=torch.int32, device=dev)
        n_cta = min((L // 128) * ((w.shape[0] + 255) // 256), sms)
        for it in range(1, a.iters + 1):
            flags[nb:] = (d // 256) * it                      # what rank 1's pushes would have raised
            counters[1] = n_cta * it
            free.fill_(it)                                    # rank 1 'has read' every earlier epoch
            base = {"n_ranks": n, "rank": 0, "chunk_rows": t, "cols": d, "n_cta": n_cta, "epoch": it, "prev_epoch": it - 1,
                    "uses": it, "push_total": n_cta * it, "consume_total": n_cta * it,
                    "gathered_ptrs": [gathered.data_ptr()] * n, "flags_ptrs": [flags.data_ptr()] * n,
                    "counters_ptrs": [counters.data_ptr()] * n, "free_ptrs": [free.data_ptr()] * n,
                    "gemm_done": done, "stats": None}
            y = lib.gemm_comm(gathered, w, None, 0, dict(base, which=1), dict(base, shard=x), None)
        torch.cuda.synchronize()
        ref = torch.cat([x, gathered[t:]]).float() @ w.float().t()
        print("gather loop-back rel err", ((y.float() - ref).norm() / ref.norm()).item())
    else:
        x, w = rnd(L, d // n), rnd(d, d // n)
        stage = torch.zeros(n, t, d, device=dev, dtype=torch.bfloat16)
        arrived = torch.zeros(8, dtype=torch.int32, device=dev)
        consumed = torch.zeros(8, dtype=torch.int32, device=dev)
        rc = torch.zeros(1, dtype=torch.int32, device=dev)
        out = torch.empty(t, d, device=dev, dtype=torch.bfloat16)
        n_cta = min((L // 128) * (d // 256), sms)
        for it in range(1, a.iters + 1):
            arrived[1] = n_cta * it                           # rank 1's tiles "arrived" (its slot holds zeros)
            consumed.fill_(it)                                # owner 1 'has reduced' every earlier epoch
            desc = {"n_ranks": n, "rank": 0, "chunk_rows": t, "epoch": it, "prev_epoch": it - 1, "uses": it,
                    "arrived_target": n_cta * it, "out": out, "stage_ptrs": [stage.data_ptr()] * n,
                    "arrived_ptrs": [arrived.data_ptr()] * n, "consumed_ptrs": [consumed.data_ptr()] * n,
                    "reduce_counter": rc}
            lib.gemm_comm(x, w, None, 0, None, None, desc)
        torch.cuda.synchronize()
        # both "owners" write into the same staging slot 0 here, so only finiteness is checked
        print("scatter loop-back finite:", bool(torch.isfinite(out.float()).all()))
    native.check_status(0)


if __name__ == "__main__":
    main()
