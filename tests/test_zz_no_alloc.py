"""The allocation-free batch-statistics entry point against the regular one.

`wb_bn2d_stats_noalloc` exists for hosts that may not allocate device memory when they need the
statistics (allocator hooks, loops with a frozen memory map).  It must give what `wb_bn2d_stats` gives,
call after call, although every call reuses one fixed scratch array that still holds the previous call's
partial sums.  Collected last on purpose: a failure here cannot hide another test's result.
"""
import ctypes

import numpy as np
import pytest

from weta_b200.core import DType, Layout
from oracle.mirror.tensor import Tensor
from weta_b200.trainer import _declare

pytestmark = pytest.mark.gpu


def test_noalloc_statistics_match_the_regular_entry_point_twice(gpu):
    lib = gpu.lib
    _declare(lib)
    P, i64, f64 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_double
    lib.wb_bn2d_stats_noalloc.argtypes = [P, P, i64, i64, i64, f64, f64, P, P, P, P]
    lib.wb_bn2d_stats_noalloc.restype = ctypes.c_int
    rng = np.random.default_rng(5)
    stream = ctypes.c_void_p(gpu.stream())
    # Two calls in a row with different shapes: the second finds the first call's partial sums in the array.
    for n, c, h, w in [(37, 24, 10, 12), (16, 130, 7, 9)]:
        x = (rng.standard_normal((n, c, h, w)) * 3 + 1.5).astype(np.float32)
        xt = Tensor.from_numpy(x, gpu)
        out = {}
        for name in ("regular", "noalloc"):
            mean, rstd = gpu.alloc(c, DType.F32), gpu.alloc(c, DType.F32)
            rm = Tensor.from_numpy(np.full(c, 0.25, np.float32), gpu)
            rv = Tensor.from_numpy(np.full(c, 2.0, np.float32), gpu)
            args = (ctypes.c_void_p(xt.storage.ptr), n, c, h * w, 1e-5, 0.1, ctypes.c_void_p(mean.ptr), ctypes.c_void_p(rstd.ptr),
                    ctypes.c_void_p(rm.storage.ptr), ctypes.c_void_p(rv.storage.ptr))
            if name == "regular":
                gpu.check(lib.wb_bn2d_stats(gpu.handle, *args))
            else:
                gpu.check(lib.wb_bn2d_stats_noalloc(stream, *args))
            fetch = lambda s: gpu.to_host(s, Layout.contiguous([c]), DType.F32)
            out[name] = (fetch(mean), fetch(rstd), rm.numpy(), rv.numpy())
        for a, b, what in zip(out["regular"], out["noalloc"], ("mean", "rstd", "running_mean", "running_var")):
            assert np.allclose(a, b, rtol=1e-6, atol=1e-7), f"{what} differs for shape {(n, c, h, w)}"
        want_mean = x.astype(np.float64).mean(axis=(0, 2, 3))
        assert np.allclose(out["noalloc"][0], want_mean, rtol=1e-5, atol=1e-5)


def test_noalloc_rejects_more_channels_than_the_fixed_array_holds(gpu):
    lib = gpu.lib
    P, i64, f64 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_double
    lib.wb_bn2d_stats_noalloc.argtypes = [P, P, i64, i64, i64, f64, f64, P, P, P, P]
    lib.wb_bn2d_stats_noalloc.restype = ctypes.c_int
    c = 40000  # more than 32768 channels; the call must fail before touching any pointer
    dummy = gpu.alloc(16, DType.F32)
    st = lib.wb_bn2d_stats_noalloc(ctypes.c_void_p(gpu.stream()), ctypes.c_void_p(dummy.ptr), 1, c, 1, 1e-5, 0.1, ctypes.c_void_p(dummy.ptr),
                                   ctypes.c_void_p(dummy.ptr), None, None)
    assert st == 1  # WB_ERR_INVALID
    assert b"32768" in lib.wb_last_error()


def _stats(gpu, lib, which, x_ptr, n, c, hw):
    mean, rstd = gpu.alloc(c, DType.F32), gpu.alloc(c, DType.F32)
    args = (ctypes.c_void_p(x_ptr), n, c, hw, 1e-5, 0.1, ctypes.c_void_p(mean.ptr), ctypes.c_void_p(rstd.ptr), None, None)
    if which == "regular":
        gpu.check(lib.wb_bn2d_stats(gpu.handle, *args))
    else:
        gpu.check(lib.wb_bn2d_stats_noalloc(ctypes.c_void_p(gpu.stream()), *args))
    fetch = lambda s: gpu.to_host(s, Layout.contiguous([c]), DType.F32)
    return fetch(mean), fetch(rstd)


def test_input_starting_at_an_odd_float_takes_the_scalar_loads(gpu):
    """Planes of whole float4s (hw % 4 == 0) but x one float past a 16-byte boundary: both entry points must read it with
    scalar loads and give the aligned result, not fault on a misaligned 128-bit load."""
    lib = gpu.lib
    _declare(lib)
    P, i64, f64 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_double
    lib.wb_bn2d_stats_noalloc.argtypes = [P, P, i64, i64, i64, f64, f64, P, P, P, P]
    lib.wb_bn2d_stats_noalloc.restype = ctypes.c_int
    rng = np.random.default_rng(11)
    n, c, h, w = 9, 6, 4, 8
    x = (rng.standard_normal(n * c * h * w) * 2 - 0.5).astype(np.float32)
    aligned = Tensor.from_numpy(x, gpu)
    shifted = Tensor.from_numpy(np.concatenate([np.zeros(1, np.float32), x]), gpu)
    want = _stats(gpu, lib, "regular", aligned.storage.ptr, n, c, h * w)
    for which in ("regular", "noalloc"):
        got = _stats(gpu, lib, which, shifted.storage.ptr + 4, n, c, h * w)
        # same sums in another order (scalar instead of 128-bit loads): equal to rounding
        assert np.allclose(got[0], want[0], rtol=1e-6, atol=1e-7) and np.allclose(got[1], want[1], rtol=1e-6, atol=1e-7), which
    # the apply kernel with the same unaligned input
    y = gpu.alloc(x.size + 1, DType.F32)
    mean, rstd = Tensor.from_numpy(want[0], gpu), Tensor.from_numpy(want[1], gpu)
    gpu.check(lib.wb_bn2d_apply(gpu.handle, P(shifted.storage.ptr + 4), n, c, h * w, P(mean.storage.ptr), P(rstd.storage.ptr), None, None, 0,
                                P(y.ptr + 4)))
    ya = gpu.alloc(x.size, DType.F32)
    gpu.check(lib.wb_bn2d_apply(gpu.handle, P(aligned.storage.ptr), n, c, h * w, P(mean.storage.ptr), P(rstd.storage.ptr), None, None, 0, P(ya.ptr)))
    got = gpu.to_host(y, Layout.contiguous([x.size + 1]), DType.F32)[1:]
    assert np.array_equal(got, gpu.to_host(ya, Layout.contiguous([x.size]), DType.F32))


def test_noalloc_at_the_channel_limit(gpu):
    """c = 32768 fills the fixed array exactly (one slab per channel)."""
    lib = gpu.lib
    _declare(lib)
    P, i64, f64 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_double
    lib.wb_bn2d_stats_noalloc.argtypes = [P, P, i64, i64, i64, f64, f64, P, P, P, P]
    lib.wb_bn2d_stats_noalloc.restype = ctypes.c_int
    rng = np.random.default_rng(12)
    n, c, hw = 2, 32768, 4
    xt = Tensor.from_numpy(rng.standard_normal(n * c * hw).astype(np.float32), gpu)
    a = _stats(gpu, lib, "regular", xt.storage.ptr, n, c, hw)
    b = _stats(gpu, lib, "noalloc", xt.storage.ptr, n, c, hw)
    assert np.allclose(a[0], b[0], rtol=1e-6, atol=1e-7) and np.allclose(a[1], b[1], rtol=1e-6, atol=1e-7)
