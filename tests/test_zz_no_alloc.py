"""The allocation-free C entry point ``lbi_rmsnorm_wgrad_noalloc``.

Some callers of the native library cannot allocate device memory at call time (a frozen memory pool, a
latency-critical loop, a plain C / ctypes host without an allocator), so this entry point carries its own
workspace.  The test drives it the way such a caller would: through the exported C symbol with raw device
pointers, twice in a row on different data, and compares with the regular entry point that takes a workspace.
The file name sorts last so that a ``-x`` run has finished every other test before it gets here.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    import lbi_b200._C as ext

    lib = ctypes.CDLL(ext.__file__)
    fn = lib.lbi_rmsnorm_wgrad_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                   ctypes.c_void_p]
    return fn


def _call(fn, d_normed, x, rstd):
    dw = torch.empty(x.shape[1], dtype=torch.float32, device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    allocations = torch.cuda.memory_stats()["allocation.all.allocated"]
    rc = fn(d_normed.data_ptr(), x.data_ptr(), rstd.data_ptr(), dw.data_ptr(), x.shape[0], x.shape[1], stream)
    assert rc == 0, f"lbi_rmsnorm_wgrad_noalloc returned {rc}"
    # the call itself must not have gone through torch's allocator
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocations
    return dw


def test_noalloc_matches_regular_entry_point_twice():
    from lbi_b200 import ops

    fn = _library()
    torch.manual_seed(11)
    for rows, dim in ((777, 1024), (50, 256)):  # second call: other sizes, stale workspace contents from the first
        g = torch.randn(rows, dim, device="cuda").bfloat16()
        x = torch.randn(rows, dim, device="cuda")
        rstd = torch.rand(rows, device="cuda") + 0.5
        got = _call(fn, g, x, rstd)
        torch.cuda.synchronize()
        want = ops.rmsnorm_wgrad(g, x, rstd)
        err = (got - want).abs()
        assert bool((err <= 1e-3 + 1e-4 * want.abs()).all()), f"max err {err.max().item():.3e}"


def test_noalloc_rejects_oversize():
    fn = _library()
    dim = 4096 + 8
    g = torch.zeros(4, dim, device="cuda", dtype=torch.bfloat16)
    x = torch.zeros(4, dim, device="cuda")
    rstd = torch.ones(4, device="cuda")
    dw = torch.empty(dim, device="cuda")
    rc = fn(g.data_ptr(), x.data_ptr(), rstd.data_ptr(), dw.data_ptr(), 4, dim, None)
    assert rc == 1  # cudaErrorInvalidValue, nothing launched
