"""Spawn gloo ranks on CPU for multi-process tests (rendezvous on 127.0.0.1)."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, args, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank))
        torch.set_num_threads(2)
        dist.init_process_group("gloo", rank=rank, world_size=world, init_method=f"tcp://127.0.0.1:{port}")
        res = fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok", res))
    except Exception:
        q.put((rank, "err", traceback.format_exc()))


def run_distributed(fn, world, *args, timeout=300):
    """Run fn(rank, world, *args) on `world` gloo ranks; returns {rank: result}; raises on any failure."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    errs = []
    try:
        for _ in range(world):
            rank, status, res = q.get(timeout=timeout)
            if status == "ok":
                out[rank] = res
            else:
                errs.append(f"rank {rank}:\n{res}")
                break
    finally:
        for p in procs:
            p.join(timeout=5 if errs else 30)
            if p.is_alive():
                p.terminate()
    if errs:
        raise AssertionError("\n".join(errs))
    return out
