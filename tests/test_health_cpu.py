"""Host-side failure detection (no GPU): heartbeats over a store, bounded barriers, rank loss between steps."""
import time

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_distributed
from odysseus_transformer_b200.utils.health import DictStore, Heartbeat, RankFailure, guarded_collective


def test_heartbeat_detects_silent_rank_with_fake_clock():
    store = DictStore()
    now = [100.0]
    hb0 = Heartbeat(store, 0, 3, timeout_s=5.0, clock=lambda: now[0], sleep=lambda s: now.__setitem__(0, now[0] + s))
    hb1 = Heartbeat(store, 1, 3, timeout_s=5.0, clock=lambda: now[0])
    hb2 = Heartbeat(store, 2, 3, timeout_s=5.0, clock=lambda: now[0])
    for hb in (hb0, hb1, hb2):
        hb.beat(0)
    assert hb0.check(0) == []
    now[0] += 10
    hb0.beat(1)
    hb1.beat(1)                        # rank 2 stays silent
    assert hb0.check(1) == [2]
    with pytest.raises(RankFailure) as e:
        hb0.barrier(1, poll_s=1.0)     # the fake sleep advances the clock past the timeout
    assert e.value.missing == [2]


def test_heartbeat_barrier_passes_when_everyone_beats():
    store = DictStore()
    hbs = [Heartbeat(store, r, 2, timeout_s=1.0) for r in range(2)]
    hbs[1].beat(7)
    hbs[0].barrier(7)


def _rank_leaves_between_steps(rank, world):
    """Rank 1 raises after step 1 (on the host, nothing in flight); rank 0 learns of it from the store before its
    next collective and raises RankFailure instead of entering an all-reduce that cannot complete."""
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, timeout_s=2.0, prefix="t/hb")
    x = torch.ones(4)
    for step in range(3):
        if rank == 1 and step == 2:
            return "left"
        hb.barrier(step)
        dist.all_reduce(x)
    return "finished"


def test_rank_leaving_between_steps_is_detected_on_gloo():
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leave_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=20)
    assert res[1] == "left"
    assert res[0].startswith("RankFailure"), res


def _leave_worker(rank, world, port, q):
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method=f"tcp://127.0.0.1:{port}",
                            timeout=datetime.timedelta(seconds=20))
    try:
        out = _rank_leaves_between_steps(rank, world)
    except RankFailure as e:
        out = f"RankFailure {e.missing}"
    q.put((rank, out))
    time.sleep(0.5)


def test_guarded_collective_maps_timeout_to_rank_failure():
    def boom():
        raise RuntimeError("[gloo] Timed out waiting 1000ms for recv operation to complete")
    with pytest.raises(RankFailure):
        guarded_collective(boom)
    def other():
        raise RuntimeError("shape mismatch")
    with pytest.raises(RuntimeError) as e:
        guarded_collective(other)
    assert not isinstance(e.value, RankFailure)
