#!/usr/bin/env python
"""Run the fused gather / scatter GEMM on ONE GPU in loop-back form, for profilers that cannot follow a
multi-rank job (``ncu`` captures one process).

The kernel is launched as rank 0 of 2 with every "peer" pointer aimed at this GPU's own buffers: the comm
warps push rank 0's shard with the same st.global path they use across NVLink, the consumers gate their
TMA loads on the same arrival counters, and the counters that rank 1 would have raised are pre-set on the
host so nothing waits for a launch that does not exist.  Numbers from this script describe the kernel's
instruction mix and on-chip behaviour, not NVLink throughput (see benchmarks/comm_bench.py for that).

    python benchmarks/fused_loopback.py gather --tokens 8192       # all-gather(x) -> QKV GEMM                 <0,1,0>
    python benchmarks/fused_loopback.py scatter --tokens 8192      # O-proj GEMM -> reduce-scatter             <0,0,1>
    python benchmarks/fused_loopback.py wgather --tokens 8192      # ZeRO-3 weight gather -> GEMM, comm warps prefetch the next weight  <0,2,0>
    python benchmarks/fused_loopback.py wgrad_rs --tokens 8192     # wgrad GEMM -> reduce-scatter              <2,0,1>
    python benchmarks/fused_loopback.py a2a --tokens 8192          # Ulysses: QKV GEMM with the all-to-all epilogue  <0,2,2>
    python benchmarks/fused_loopback.py ring_push --tokens 8192    # attention forward whose comm warps push K/V (ring step)
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gather", "scatter", "wgather", "wgrad_rs", "a2a", "ring_push"])
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

    class Slot:
        """Buffers of one gather slot with both "ranks" mapped onto this GPU."""

        def __init__(self, chunk_rows, cols):
            self.chunk_rows, self.cols = chunk_rows, cols
            self.gathered = rnd(n * chunk_rows, cols)
            self.unit = 128 if chunk_rows % 128 == 0 else 64
            self.nb = chunk_rows // self.unit
            self.flags = torch.zeros(n * self.nb, dtype=torch.int32, device=dev)
            self.counters = torch.zeros(8, dtype=torch.int32, device=dev)
            self.free = torch.zeros(8, dtype=torch.int32, device=dev)
            self.done = torch.zeros(1, dtype=torch.int32, device=dev)

        def desc(self, it, n_cta, arrived_ranks, **extra):
            """Description of epoch ``it``; the row blocks of ``arrived_ranks`` are marked as already delivered."""
            per_block = (self.cols // (256 if self.cols % 256 == 0 else 64)) * it
            for p in arrived_ranks:
                self.flags[p * self.nb:(p + 1) * self.nb] = per_block
                self.counters[p] = n_cta * it
            self.free.fill_(it)
            dd = {"n_ranks": n, "rank": 0, "chunk_rows": self.chunk_rows, "cols": self.cols, "n_cta": n_cta, "epoch": it,
                  "prev_epoch": it - 1, "uses": it, "push_total": n_cta * it, "consume_total": n_cta * it,
                  "gathered_ptrs": [self.gathered.data_ptr()] * n, "flags_ptrs": [self.flags.data_ptr()] * n,
                  "counters_ptrs": [self.counters.data_ptr()] * n, "free_ptrs": [self.free.data_ptr()] * n,
                  "gemm_done": self.done, "stats": None}
            dd.update(extra)
            return dd

    if a.what == "wgather":
        # x [t, d] @ gather(W)^T with W [2 * 11008, d] sharded on rows; the comm warps push the NEXT weight's shard meanwhile
        I = 11008
        x = rnd(t, d)
        cur, nxt = Slot(2 * I // n, d), Slot(d // n, I)
        nxt_shard = rnd(d // n, I)
        n_cta = min(((t + 127) // 128) * ((2 * I + 255) // 256), sms)
        for it in range(1, a.iters + 1):
            y = lib.gemm_comm(x, cur.gathered, None, 0, cur.desc(it, n_cta, [0, 1], which=2),
                              nxt.desc(it, n_cta, [1], shard=nxt_shard), None)
        torch.cuda.synchronize()
        ref = x.float() @ cur.gathered.float().t()
        print("weight-gather loop-back rel err", ((y.float() - ref).norm() / ref.norm()).item(),
              "| prefetched shard delivered:", bool(torch.equal(nxt.gathered[:d // n], nxt_shard)))
    elif a.what == "wgrad_rs":
        # dW [2I, d] = dy^T x, rows reduce-scattered over the 2 "ranks"
        I = 11008
        dy, x = rnd(t, 2 * I), rnd(t, d)
        chunk = 2 * I // n
        stage = torch.zeros(n, chunk, d, device=dev, dtype=torch.bfloat16)
        arrived = torch.zeros(8, dtype=torch.int32, device=dev)
        consumed = torch.zeros(8, dtype=torch.int32, device=dev)
        rc = torch.zeros(1, dtype=torch.int32, device=dev)
        out = torch.empty(chunk, d, device=dev, dtype=torch.bfloat16)
        n_cta = min(((2 * I + 127) // 128) * (d // 256), sms)
        for it in range(1, a.iters + 1):
            arrived[1] = n_cta * it
            consumed.fill_(it)
            desc = {"n_ranks": n, "rank": 0, "chunk_rows": chunk, "epoch": it, "prev_epoch": it - 1, "uses": it,
                    "arrived_target": n_cta * it, "out": out, "stage_ptrs": [stage.data_ptr()] * n,
                    "arrived_ptrs": [arrived.data_ptr()] * n, "consumed_ptrs": [consumed.data_ptr()] * n, "reduce_counter": rc}
            lib.gemm_comm(dy, x, None, 2, None, None, desc)
        torch.cuda.synchronize()
        print("wgrad reduce-scatter loop-back finite:", bool(torch.isfinite(out.float()).all()))
    elif a.what == "a2a":
        # Ulysses QKV projection: column group u of x @ gather(W)^T goes to rank u's [Tb, G] receive buffer at rows r * t
        hq = hkv = 16
        G = (hq + 2 * hkv) * 128
        x = rnd(t, d)
        wslot = Slot(n * G // n, d)
        recv = torch.zeros(n * t, G, device=dev, dtype=torch.bfloat16)
        arrived = torch.zeros(8, dtype=torch.int32, device=dev)
        consumed = torch.zeros(8, dtype=torch.int32, device=dev)
        dummy = torch.zeros(1, dtype=torch.int32, device=dev)
        n_cta = min(((t + 127) // 128) * ((n * G + 255) // 256), sms)
        for it in range(1, a.iters + 1):
            consumed.fill_(it)
            sc = {"mode": 2, "n_ranks": n, "rank": 0, "chunk_rows": 0, "epoch": it, "prev_epoch": it - 1, "uses": it,
                  "arrived_target": n_cta * it, "out": recv, "stage_ptrs": [recv.data_ptr()] * n,
                  "arrived_ptrs": [arrived.data_ptr()] * n, "consumed_ptrs": [consumed.data_ptr()] * n, "reduce_counter": dummy,
                  "a2a_cols": G, "a2a_ld": G, "a2a_row0": 0, "a2a_col0": 0}
            lib.gemm_comm(x, wslot.gathered, None, 0, wslot.desc(it, n_cta, [0, 1], which=2), None, sc)
        torch.cuda.synchronize()
        # both column groups land in rows [0, t) of the one buffer; the second group is written last by most tiles
        print("all-to-all epilogue loop-back finite:", bool(torch.isfinite(recv[:t].float()).all()),
              "| arrival count", int(arrived[0].item()))
    elif a.what == "ring_push":
        # one ring step: causal attention on the local block while the comm warps push this rank's packed K|V rows downstream
        hq = hkv = 8
        qkv = rnd(t, hq + 2 * hkv, 128)
        q, k, v = qkv[:, :hq], qkv[:, hq:hq + hkv], qkv[:, hq + hkv:]
        shard = torch.as_strided(k, (t, 2 * hkv * 128), (k.stride(0), 1))
        slot = Slot(t, 2 * hkv * 128)
        n_push = int(lib.attn_fwd_ctas(t, hq))
        for it in range(1, a.iters + 1):
            o, lse = lib.attn_fwd_push(q, k, v, True, 128 ** -0.5, slot.desc(it, n_push, [], shard=shard, dest_first=1, dest_count=1))
        torch.cuda.synchronize()
        o2, _ = lib.attn_fwd(q, k, v, True, 128 ** -0.5)
        print("ring-step loop-back: attention equal to the plain kernel:", bool(torch.equal(o, o2)),
              "| K|V delivered:", bool(torch.equal(slot.gathered[:t], shard)))
    elif a.what == "gather":
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
