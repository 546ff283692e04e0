"""The allocation-free column sum, called through its exported C symbol.

It serves callers that hand the library raw device pointers and may not allocate (a fixed memory
budget, their own memory manager, a thread that must stay away from allocators).  The result must
equal the regular entry point's, on two calls in a row (the second call reuses the library's fixed
scratch array with the first call's leftovers in it).  This file sorts last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from infinitrain_b200 import _ext

    mod = _ext.load(required=True)
    lib = ctypes.CDLL(mod.__file__)
    fn = lib.itb_colsum_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_void_p]
    return mod, fn


def _call(fn, x, out, accumulate=0):
    dtype = 1 if x.dtype == torch.bfloat16 else 0
    stream = torch.cuda.current_stream().cuda_stream
    return fn(x.data_ptr(), dtype, x.stride(0), out.data_ptr(), x.shape[0], x.shape[1], accumulate, stream)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_colsum_matches_regular_entry_point(dtype):
    mod, fn = _lib()
    torch.manual_seed(0)
    # first call outside any stream capture: it looks up the scratch array's device address
    x1 = torch.randn(4000, 776, device="cuda").to(dtype)
    x2 = torch.randn(1000, 2304, device="cuda").to(dtype)     # different shape: stale partials around
    for x in (x1, x2):
        out = torch.full((x.shape[1],), float("nan"), device="cuda")
        assert _call(fn, x, out) == 0
        torch.cuda.synchronize()
        ref = mod.colsum(x)
        assert torch.allclose(out, ref, rtol=1e-4, atol=1e-4), (out - ref).abs().max().item()
        assert (out - x.float().sum(0)).norm() / x.float().sum(0).norm() < 1e-4
    # accumulate mode
    out = torch.ones(x2.shape[1], device="cuda")
    assert _call(fn, x2, out, accumulate=1) == 0
    torch.cuda.synchronize()
    assert torch.allclose(out, mod.colsum(x2) + 1, rtol=1e-4, atol=1e-4)


def test_static_scratch_rejects_oversized_requests():
    _, fn = _lib()
    # ceil(rows/128) * N > 1 Mi partial sums; the pointers are never touched on this path
    x = torch.empty(8, 8, device="cuda")
    out = torch.zeros(8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(x.data_ptr(), 0, 8192, out.data_ptr(), 128 * 200, 8192, 0, stream)
    assert rc == -100
    assert fn(x.data_ptr(), 0, 12, out.data_ptr(), 8, 12, 0, stream) == -3      # N not a multiple of 8
    # more than 65535 row blocks (the grid's y limit) passes the scratch check with N = 8: rejected, not launched
    assert fn(x.data_ptr(), 0, 8, out.data_ptr(), 65536 * 128, 8, 0, stream) == -3
    assert fn(x.data_ptr(), 0, 8, out.data_ptr(), 8, 16, 0, stream) == -3       # row stride shorter than a row
    assert fn(x.data_ptr() + 4, 0, 8, out.data_ptr(), 8, 8, 0, stream) == -3    # x not 16-byte aligned
