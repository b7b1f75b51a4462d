"""The allocation-free RMSNorm backward, called the way a plain C host would call it.

``ody_rmsnorm_bwd_noalloc`` serves callers that cannot (or may not) allocate device memory: its scratch
is a fixed array inside the library.  The test goes through the exported C symbol with raw pointers,
several times in a row with different shapes and inputs, and checks each result against the regular entry
point (which takes its workspace from PyTorch's allocator) and against a plain fp32 PyTorch evaluation of the
same formula, within the tolerances of the other kernel tests.  Bad pointers and sizes must come back as error
codes without a launch.  It runs last so that a failure here cannot hide results of any other test."""
import ctypes
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _load():
    import odysseus_transformer_b200
    from odysseus_transformer_b200.ops import native
    lib = native.lib()                      # makes sure libtorch and the extension are loaded
    path = os.path.join(os.path.dirname(odysseus_transformer_b200.__file__), "_C.so")
    cdll = ctypes.CDLL(path)
    fn = cdll.ody_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
    err = cdll.ody_noalloc_strerror
    err.restype = ctypes.c_char_p
    err.argtypes = [ctypes.c_int]
    return lib, fn, err


def _rand(*shape):
    return torch.randn(*shape, device="cuda", dtype=torch.float32).to(torch.bfloat16)


def _one_call(lib, fn, rows, dim, with_ds):
    dy, x, w = _rand(rows, dim), _rand(rows, dim), _rand(dim) + 1
    ds = _rand(rows, dim) if with_ds else None
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    dx = torch.empty_like(x)
    dw = torch.empty(dim, device="cuda", dtype=torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), ds.data_ptr() if with_ds else None,
            dx.data_ptr(), dw.data_ptr(), rows, dim, stream)
    assert rc == 0, rc
    dx_ref, dw_ref = lib.rmsnorm_bwd(dy, x, w, rstd, ds)
    torch.cuda.synchronize()
    torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dw, dw_ref, rtol=1e-3, atol=1e-2 * math.sqrt(rows))
    # the same op in plain fp32 PyTorch (ops/torch_ref.py is the oracle of every kernel test)
    from odysseus_transformer_b200.ops import torch_ref
    dx32, dw32 = torch_ref.rmsnorm_bwd(dy.float(), x.float(), w.float(), rstd)
    if with_ds:
        dx32 = dx32 + ds.float()
    torch.testing.assert_close(dx.float(), dx32, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dw, dw32.float(), rtol=1e-3, atol=1e-2 * math.sqrt(rows))


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    torch.cuda.set_device(0)
    lib, fn, err = _load()
    torch.manual_seed(0)
    _one_call(lib, fn, 1000, 4096, with_ds=False)
    # second call: fewer rows than blocks of the first call, narrower rows, residual gradient added -
    # whatever the first call left in the shared scratch must not show up here
    _one_call(lib, fn, 37, 1024, with_ds=True)
    _one_call(lib, fn, 4096, 8192, with_ds=True)


def test_noalloc_rejects_sizes_beyond_the_built_in_scratch():
    torch.cuda.set_device(0)
    lib, fn, err = _load()
    x = _rand(8, 16384)
    rstd = torch.ones(8, device="cuda")
    dw = torch.empty(16384, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), rstd.data_ptr(), None, x.data_ptr(), dw.data_ptr(), 8, 16384,
            torch.cuda.current_stream().cuda_stream)
    assert rc == 9001
    assert b"exceeds" in err(rc)
    assert fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), rstd.data_ptr(), None, x.data_ptr(), dw.data_ptr(), 8, 12,
              torch.cuda.current_stream().cuda_stream) == 9002


def test_noalloc_refuses_bad_pointers_and_handles_zero_rows():
    """Null or misaligned buffers are answered with an error code on the host (the kernels use 16-byte accesses and
    would fault on them); zero rows is a valid call that only clears dw."""
    torch.cuda.set_device(0)
    lib, fn, err = _load()
    rows, dim = 16, 256
    dy, x, w = _rand(rows, dim), _rand(rows, dim), _rand(dim)
    rstd = torch.ones(rows, device="cuda")
    dx = torch.empty_like(x)
    dw = torch.full((dim,), 7.0, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    good = [dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dw.data_ptr()]
    for i in (0, 1, 2, 3, 5, 6):                      # each required pointer null in turn
        a = list(good)
        a[i] = None
        assert fn(*a, rows, dim, st) == 9003, i
    for i in (0, 1, 2, 4, 5):                         # 2 bytes off a 16-byte boundary
        a = list(good)
        a[i] = x.data_ptr() + 2
        assert fn(*a, rows, dim, st) == 9003, i
    a = list(good)
    a[6] = dw.data_ptr() + 2
    assert fn(*a, rows, dim, st) == 9003
    assert b"aligned" in err(9003)
    torch.cuda.synchronize()
    assert torch.all(dw == 7.0)                        # nothing ran
    assert fn(None, None, None, None, None, None, dw.data_ptr(), 0, dim, st) == 0
    torch.cuda.synchronize()
    assert torch.all(dw == 0.0)
    assert fn(*good, rows, dim, st) == 0               # and the entry point still works afterwards
    torch.cuda.synchronize()
    assert torch.isfinite(dx.float()).all() and torch.isfinite(dw).all()
