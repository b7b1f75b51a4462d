"""Host-side failure detection: heartbeats and bounded barriers over a key-value store.

The reference has no failure handling at all - a lost rank leaves the others blocked inside NCCL
(reference ``train.py:56-57`` sets no timeout; ``run.sh:24`` is plain torchrun).  Here every rank
publishes a heartbeat (step number + wall time) to the rendezvous store between steps, checks its
peers' heartbeats before launching the next step's collectives, and raises ``RankFailure`` naming the
silent ranks instead of entering a collective that cannot complete.  Nothing here touches a GPU:
detection happens between steps, with no kernel or collective in flight.  Recovery is a restart from
the last checkpoint; because checkpoints are unsharded HF state dicts the restart may use a
different world size.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional


class RankFailure(RuntimeError):
    def __init__(self, missing: List[int], detail: str = ""):
        super().__init__(f"ranks {missing} stopped responding {detail}".strip())
        self.missing = missing


class DictStore:
    """In-process stand-in for ``torch.distributed.Store`` (tests and single-process runs)."""

    def __init__(self):
        self.kv: Dict[str, bytes] = {}

    def set(self, k: str, v) -> None:
        self.kv[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        return self.kv[k]

    def check(self, keys) -> bool:
        return all(k in self.kv for k in keys)

    def add(self, k: str, n: int) -> int:
        cur = int(self.kv.get(k, b"0")) + n
        self.kv[k] = str(cur).encode()
        return cur


class Heartbeat:
    """Per-rank liveness record in a shared store.

    ``beat(step)`` publishes; ``check(step)`` returns the ranks whose last published step is older
    than ``step - max_lag`` *and* whose last beat is older than ``timeout_s``; ``barrier(step)`` waits
    (bounded) until every rank has published ``step`` and raises ``RankFailure`` otherwise."""

    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 30.0, prefix: str = "ody/hb",
                 clock=time.time, sleep=time.sleep):
        self.store, self.rank, self.world = store, rank, world_size
        self.timeout_s, self.prefix = timeout_s, prefix
        self.clock, self.sleep = clock, sleep

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step}:{self.clock():.3f}")

    def read(self, r: int) -> Optional[tuple]:
        if not self.store.check([self._key(r)]):
            return None
        s, t = self.store.get(self._key(r)).decode().split(":")
        return int(s), float(t)

    def check(self, step: int, max_lag: int = 0) -> List[int]:
        now, missing = self.clock(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            rec = self.read(r)
            if rec is None or (rec[0] < step - max_lag and now - rec[1] > self.timeout_s):
                missing.append(r)
        return missing

    def barrier(self, step: int, poll_s: float = 0.01) -> None:
        self.beat(step)
        deadline = self.clock() + self.timeout_s
        while True:
            behind = [r for r in range(self.world)
                      if r != self.rank and ((self.read(r) or (-1, 0.0))[0] < step)]
            if not behind:
                return
            if self.clock() >= deadline:
                raise RankFailure(behind, f"(no heartbeat for step {step} within {self.timeout_s}s)")
            self.sleep(poll_s)


def guarded_collective(fn, *args, on_timeout: str = "collective timed out", **kw):
    """Run a torch.distributed call and turn its timeout / peer-loss error into ``RankFailure``."""
    try:
        return fn(*args, **kw)
    except RuntimeError as e:   # gloo: "Timed out waiting", "Connection closed by peer"; NCCL watchdog errors
        msg = str(e)
        if any(s in msg for s in ("Timed out", "timed out", "Connection closed", "Connection reset", "NCCL", "peer")):
            raise RankFailure([], f"({on_timeout}: {msg.splitlines()[0][:200]})") from e
        raise
