#!/usr/bin/env python
"""What NVLink gives to plain in-kernel peer loads / stores, as a function of how many SMs take part.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29530 benchmarks/p2p_bench.py

Every rank copies 256 MiB between its own buffer and its right neighbour's symmetric buffer with
``peer_copy`` (16-byte accesses, 8 in flight per thread) - ``push`` = local loads + peer stores,
``pull`` = peer loads + local stores - for several grid sizes.  CUDA-event timing, max over ranks.
These numbers size the comm warps of the fused gather GEMM (csrc/gemm_comm.cu)."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from odysseus_transformer_b200.comm.symm import SymmetricHeap
    from odysseus_transformer_b200.mesh import init_parallel_context
    from odysseus_transformer_b200.ops import native
    native.set_backend("fused")
    ctx = init_parallel_context("odysseus", backend="fused")
    lib = native.lib()
    n, rank, dev = ctx.world_size, ctx.rank, ctx.device
    nbytes = 256 << 20
    heap = SymmetricHeap(ctx.world_group, dev, nbytes + (1 << 20))
    off = heap.alloc(nbytes)
    local = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    peer = (rank + 1) % n
    for mode in ("push", "pull"):
        for ctas, threads in [(8, 256), (16, 512), (32, 512), (64, 512), (148, 128), (148, 512), (296, 512)]:
            dst, src = (heap.ptr(peer, off), local.data_ptr()) if mode == "push" else (local.data_ptr(), heap.ptr(peer, off))
            for _ in range(2):
                lib.peer_copy(dst, src, nbytes, ctas, threads)
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(4):
                lib.peer_copy(dst, src, nbytes, ctas, threads)
            e1.record()
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1) / 4], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            if rank == 0:
                gbs = nbytes / ms.item() / 1e6
                print(json.dumps({"mode": mode, "ctas": ctas, "threads": threads, "ms": round(ms.item(), 4),
                                  "GB_per_s": round(gbs, 1), "GB_per_s_per_cta": round(gbs / ctas, 2)}), flush=True)
            dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
