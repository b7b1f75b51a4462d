"""Device-side failure detection: a wait that nothing satisfies ends in a status code, not a hang.

The fused gather GEMM waits on arrival counters that other ranks raise.  Here, on one GPU, a consumer is
launched for an operand that nobody ever pushes (the counters stay zero): every wait inside the kernel is
bounded (about a second of SM clocks), after which the kernel records ``ODY_ERR_TIMEOUT_PEER`` (105) in the
status word, drains, frees its TMEM and returns.  The context stays usable: a normal GEMM runs right after."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_unsatisfied_peer_wait_reports_status_and_returns():
    from odysseus_transformer_b200.ops import native
    native.set_backend("fused")
    lib = native.lib()
    dev = torch.device("cuda", 0)
    lib.clear_status(0)
    lib.set_peer_wait_limit(1_000_000_000)        # ~0.5 s instead of the 10 s default, to keep the test short
    n, chunk, cols, N = 2, 128, 256, 256
    gathered = torch.zeros(n * chunk, cols, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, cols, device=dev).to(torch.bfloat16)
    flags = torch.zeros(64, dtype=torch.int32, device=dev)        # arrival counters nobody raises
    counters = torch.zeros(8, dtype=torch.int32, device=dev)
    free = torch.zeros(8, dtype=torch.int32, device=dev)
    done = torch.zeros(1, dtype=torch.int32, device=dev)
    consume = {"which": 1, "n_ranks": n, "rank": 0, "chunk_rows": chunk, "cols": cols, "n_cta": 2, "epoch": 1,
               "prev_epoch": 0, "uses": 1, "push_total": 2, "consume_total": 2,
               "gathered_ptrs": [gathered.data_ptr()] * n, "flags_ptrs": [flags.data_ptr()] * n,
               "counters_ptrs": [counters.data_ptr()] * n, "free_ptrs": [free.data_ptr()] * n,
               "gemm_done": done, "stats": None}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    lib.gemm_comm(gathered, w, None, 0, consume, None, None)
    e1.record()
    torch.cuda.synchronize()
    assert e0.elapsed_time(e1) < 10_000, "the bounded wait did not end in time"
    assert lib.status(0) == 105
    lib.set_peer_wait_limit(20_000_000_000)
    with pytest.raises(RuntimeError):
        native.check_status(0)
    assert lib.status(0) == 0
    # the context is intact
    a = torch.randn(256, 128, device=dev).to(torch.bfloat16)
    c = lib.gemm(a, a, None, 0, False)
    torch.cuda.synchronize()
    ref = a.float() @ a.float().t()
    assert ((c.float() - ref).norm() / ref.norm()).item() < 5e-3
    assert lib.status(0) == 0
