"""Multi-GPU parity: every mode on 2 (or 4) B200s against a single-GPU run of the same weights."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(n, *args, timeout=600):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(_port()), os.path.join(HERE, "mgpu_worker.py"), *map(str, args)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "RESULT" in r.stdout, tail
    print(r.stdout[-600:])
    return r.stdout


@pytest.mark.parametrize("backend", ["library", "fused"])
@pytest.mark.parametrize("mode", ["odysseus", "tpsp", "ulysses", "ring"])
def test_modes_2gpu(mode, backend):
    _launch(2, mode, "small", 1024, 0, 1, backend)


def test_shard_rows_with_tile_edges_2gpu():
    """L / N = 192: shard boundaries fall inside 128-row tiles of the fused GEMMs (64-row units on the wire)."""
    _launch(2, "odysseus", "small", 384, 0, 1, "fused", 2)
    _launch(2, "tpsp", "small", 384, 0, 1, "fused", 2)


@pytest.mark.parametrize("mode", ["odysseus", "ulysses", "ring"])
def test_five_iterations_reuse_every_slot_2gpu(mode):
    """Both buffers of every slot pair are reused several times; the cumulative arrival targets keep growing."""
    _launch(2, mode, "small", 1024, 0, 1, "fused", 5)


@pytest.mark.parametrize("variant", ["zero2", "gradckpt", "chunked"])
def test_optional_modes_fused_2gpu(variant):
    _launch(2, "odysseus", "small", 1024, 0, 1, "fused", 3, variant)


def test_ulysses_4gpu():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    _launch(4, "ulysses", "small", 2048, 0, 1, "fused")


def test_ring_4gpu():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    _launch(4, "ring", "small-gqa", 2048, 0, 1, "fused")


@pytest.mark.parametrize("mode", ["odysseus", "ulysses"])
def test_hybrid_4gpu(mode):
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    _launch(4, mode, "small-gqa", 1024, 2, 2, "fused")
