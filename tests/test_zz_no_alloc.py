"""The allocation-free column sum (``nb_colsum_noalloc``), called through its exported C symbol.

Collected last on purpose (file name): the library's built-in scratch array must behave the
same in a fresh process and after every other test has used the device.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_COLS = 8192
ERR_TOO_WIDE, ERR_BAD_SHAPE = -1, -2


def _entry():
    from nabla_b200.native import load

    lib = load("libnb_noalloc.so")
    fn = lib.nb_colsum_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p]
    lib.nb_noalloc_strerror.restype = ctypes.c_char_p
    lib.nb_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib, fn


def _call(fn, x, out):
    dt = {torch.float32: 0, torch.bfloat16: 1}
    return fn(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], dt[x.dtype], dt[out.dtype],
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_colsum_matches_regular_entry_point_twice(dtype):
    from nabla_b200.native import kernels

    lib, fn = _entry()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    warm = torch.zeros(8, 8, device=dev, dtype=dtype)
    assert _call(fn, warm, torch.empty(8, device=dev)) == 0        # set-up call: module load + address look-up
    torch.cuda.synchronize()
    # two calls in a row; the second is smaller, so it runs over scratch that still holds the
    # first call's partial sums
    for rows, n in ((5000, 2048), (777, 264)):
        x = torch.randn(rows, n, device=dev, dtype=dtype)
        want = kernels.colsum(x, out_dtype=torch.float32)          # the existing entry point
        out = torch.empty(n, device=dev, dtype=torch.float32)      # allocated by the caller, before the call
        torch.cuda.synchronize()
        before = torch.cuda.memory_stats(dev)["allocation.all.allocated"]
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc = _call(fn, x, out)
        free_after = torch.cuda.mem_get_info(dev)[0]
        after = torch.cuda.memory_stats(dev)["allocation.all.allocated"]
        assert rc == 0, lib.nb_noalloc_strerror(rc)
        assert after == before                                      # nothing asked of torch's allocator
        assert free_after >= free_before                            # and nothing taken from the driver either
        torch.cuda.synchronize()
        ref = x.float().sum(0)
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-3
        torch.testing.assert_close(out, want, rtol=tol, atol=tol)
        torch.testing.assert_close(out, ref, rtol=tol, atol=tol * (rows ** 0.5))


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_no_alloc_colsum_rejects_what_does_not_fit():
    lib, fn = _entry()
    dev = torch.device("cuda", 0)
    x = torch.zeros(4, MAX_COLS + 8, device=dev, dtype=torch.float32)
    out = torch.full((MAX_COLS + 8,), 7.0, device=dev)
    assert _call(fn, x, out) == ERR_TOO_WIDE
    assert b"8192" in lib.nb_noalloc_strerror(ERR_TOO_WIDE)
    y = torch.zeros(4, 6, device=dev, dtype=torch.float32)       # 6 columns: rows are not 16-byte vectors
    assert _call(fn, y, out) == ERR_BAD_SHAPE
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())                               # rejected calls launched nothing
