"""ctypes binding of libweta_b200.so: the CUDA backend object.

`B200Backend` has the method set of `weta_core::Backend` (crates/weta-core/src/backend.rs:65-106)
and is what `Tensor` dispatches to, the way `Storage::Cuda` dispatches to `weta_cuda::backend(i)`
in crates/weta-tensor/src/storage.rs:83-119.  There is no fallback: if the shared library is
missing or no sm_100 device is present, construction raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np

from .core import Distribution, DType, Im2ColParams, Layout, WbView

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libweta_b200.so")


class WbConvParams(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("kh", "kw", "sh", "sw", "ph", "pw", "dh", "dw")]


class BackendError(RuntimeError):
    """A non-zero WbStatus.  The reference panics at the same places (e.g. crates/weta-cuda/src/lib.rs:207, 518)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"weta_b200 status {status}: {message}")
        self.status = status


_lib = None


def load_library():
    """Loads libweta_b200.so once and declares every entry point of include/weta_b200.h."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise BackendError(5, f"{LIB_PATH} is missing: build it with `make -C weta_b200/csrc` (no CPU fallback exists)")
    lib = ctypes.CDLL(LIB_PATH)
    P, PP = ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)
    V = ctypes.POINTER(WbView)
    C = ctypes.POINTER(WbConvParams)
    i32, i64, f64, u64 = ctypes.c_int, ctypes.c_int64, ctypes.c_double, ctypes.c_uint64
    sig = {
        "wb_device_count": ([], i32),
        "wb_backend_create": ([i32, PP], i32),
        "wb_backend_create_on_stream": ([i32, P, PP], i32),
        "wb_backend_destroy": ([P], i32),
        "wb_backend_ordinal": ([P], i32),
        "wb_backend_stream": ([P], P),
        "wb_synchronize": ([P], i32),
        "wb_last_error": ([], ctypes.c_char_p),
        "wb_set_profiling": ([P, i32], i32),
        "wb_profile_report": ([P], ctypes.c_char_p),
        "wb_set_matmul_mode": ([P, i32], i32),
        "wb_get_matmul_mode": ([P], i32),
        "wb_launch_count": ([P], i64),
        "wb_alloc": ([P, i64, i32, PP], i32),
        "wb_zeros": ([P, i64, i32, PP], i32),
        "wb_free": ([P, P], i32),
        "wb_storage_wrap": ([P, P, i64, i32, PP], i32),
        "wb_storage_data": ([P], P),
        "wb_storage_len": ([P], i64),
        "wb_storage_dtype": ([P], i32),
        "wb_from_host": ([P, P, i64, i32, PP], i32),
        "wb_to_host": ([P, V, P], i32),
        "wb_upload_async": ([P, P, P, i64], i32),
        "wb_download_async": ([P, P, P, i64], i32),
        "wb_arena_bytes_reserved": ([P], i64),
        "wb_copy_strided": ([P, V, V], i32),
        "wb_unary": ([P, i32, f64, f64, V, PP], i32),
        "wb_unary_into": ([P, i32, f64, f64, V, P], i32),
        "wb_binary": ([P, i32, V, V, PP], i32),
        "wb_binary_into": ([P, i32, V, V, P], i32),
        "wb_reduce": ([P, i32, V, i32, PP], i32),
        "wb_reduce_into": ([P, i32, V, i32, P], i32),
        "wb_matmul": ([P, V, V, PP], i32),
        "wb_matmul_into": ([P, V, V, P], i32),
        "wb_im2col": ([P, V, C, PP], i32),
        "wb_im2col_into": ([P, V, C, P], i32),
        "wb_col2im": ([P, V, C, i64, i64, i64, PP], i32),
        "wb_col2im_into": ([P, V, C, i64, i64, i64, P], i32),
        "wb_cast": ([P, V, i32, PP], i32),
        "wb_cast_into": ([P, V, i32, P], i32),
        "wb_random": ([P, i64, i32, i32, f64, f64, u64, PP], i32),
        "wb_random_into": ([P, i64, i32, i32, f64, f64, u64, P], i32),
        "wb_splitmix64": ([u64, u64], u64),
        "wb_gemm_check": ([P], i32),
    }
    for name, (args, res) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, res
    _lib = lib
    return lib


class DeviceStorage:
    """An owned WbStorage handle; returns its block to the backend's arena when collected."""

    __slots__ = ("handle", "backend", "__weakref__")

    def __init__(self, handle: int, backend: "B200Backend"):
        self.handle = handle
        self.backend = backend

    @property
    def ptr(self) -> int:
        return self.backend.lib.wb_storage_data(self.handle)

    @property
    def length(self) -> int:
        return self.backend.lib.wb_storage_len(self.handle)

    def __del__(self):
        be = self.backend
        if self.handle and be is not None and be.handle:
            be.lib.wb_free(be.handle, self.handle)
            self.handle = None


class B200Backend:
    """One per GPU ordinal (crates/weta-cuda/src/lib.rs:129-146)."""

    name = "b200"

    def __init__(self, ordinal: int = 0, stream: Optional[int] = None):
        self.lib = load_library()
        self.handle = None
        out = ctypes.c_void_p()
        if stream is None:
            st = self.lib.wb_backend_create(ordinal, ctypes.byref(out))
        else:
            st = self.lib.wb_backend_create_on_stream(ordinal, ctypes.c_void_p(stream), ctypes.byref(out))
        if st != 0:
            raise BackendError(st, self.lib.wb_last_error().decode())
        self.handle = out.value
        self.ordinal = ordinal

    def close(self):
        if self.handle:
            self.lib.wb_backend_destroy(self.handle)
            self.handle = None

    # -- helpers ----------------------------------------------------------------------------
    def check(self, status: int):
        if status != 0:
            raise BackendError(status, self.lib.wb_last_error().decode())

    def _wrap(self, out: ctypes.c_void_p) -> DeviceStorage:
        return DeviceStorage(out.value, self)

    @staticmethod
    def _view(s: DeviceStorage, l: Layout, dt: int) -> WbView:
        return l.view(s.ptr, dt)

    def synchronize(self):
        self.check(self.lib.wb_synchronize(self.handle))

    def stream(self) -> int:
        return self.lib.wb_backend_stream(self.handle) or 0

    def launch_count(self) -> int:
        return self.lib.wb_launch_count(self.handle)

    def gemm_check(self):
        """Raises if a tensor-core kernel gave up on a pipeline barrier since the last check."""
        self.check(self.lib.wb_gemm_check(self.handle))

    def set_matmul_mode(self, mode: int):
        self.check(self.lib.wb_set_matmul_mode(self.handle, mode))

    def set_profiling(self, on: bool):
        self.check(self.lib.wb_set_profiling(self.handle, int(on)))

    def profile_report(self) -> str:
        return self.lib.wb_profile_report(self.handle).decode()

    def alloc(self, n: int, dt: int) -> DeviceStorage:
        out = ctypes.c_void_p()
        self.check(self.lib.wb_alloc(self.handle, n, dt, ctypes.byref(out)))
        return self._wrap(out)

    def wrap_pointer(self, ptr: int, n: int, dt: int) -> DeviceStorage:
        out = ctypes.c_void_p()
        self.check(self.lib.wb_storage_wrap(self.handle, ctypes.c_void_p(ptr), n, dt, ctypes.byref(out)))
        return self._wrap(out)

    # -- trait surface ----------------------------------------------------------------------
    def from_host(self, flat: np.ndarray) -> DeviceStorage:
        flat = np.ascontiguousarray(flat)
        out = ctypes.c_void_p()
        self.check(self.lib.wb_from_host(self.handle, flat.ctypes.data, flat.size, DType.of(flat), ctypes.byref(out)))
        return self._wrap(out)

    def to_host(self, s: DeviceStorage, l: Layout, dt: int) -> np.ndarray:
        out = np.empty(l.numel(), dtype=DType.np(dt))
        v = self._view(s, l, dt)
        self.check(self.lib.wb_to_host(self.handle, ctypes.byref(v), out.ctypes.data))
        return out

    def zeros(self, n: int, dt: int) -> DeviceStorage:
        out = ctypes.c_void_p()
        self.check(self.lib.wb_zeros(self.handle, n, dt, ctypes.byref(out)))
        return self._wrap(out)

    def copy_strided(self, src: DeviceStorage, ls: Layout, dt: int, dst: DeviceStorage, ld: Layout) -> None:
        vs, vd = self._view(src, ls, dt), self._view(dst, ld, dt)
        self.check(self.lib.wb_copy_strided(self.handle, ctypes.byref(vs), ctypes.byref(vd)))

    def unary(self, op: int, p1: float, p2: float, s: DeviceStorage, l: Layout, dt: int) -> DeviceStorage:
        out, v = ctypes.c_void_p(), self._view(s, l, dt)
        self.check(self.lib.wb_unary(self.handle, op, p1, p2, ctypes.byref(v), ctypes.byref(out)))
        return self._wrap(out)

    def binary(self, op: int, sa, la: Layout, sb, lb: Layout, dt: int) -> DeviceStorage:
        out, va, vb = ctypes.c_void_p(), self._view(sa, la, dt), self._view(sb, lb, dt)
        self.check(self.lib.wb_binary(self.handle, op, ctypes.byref(va), ctypes.byref(vb), ctypes.byref(out)))
        return self._wrap(out)

    def reduce(self, op: int, s, l: Layout, dt: int, axis: int) -> DeviceStorage:
        out, v = ctypes.c_void_p(), self._view(s, l, dt)
        self.check(self.lib.wb_reduce(self.handle, op, ctypes.byref(v), axis, ctypes.byref(out)))
        return self._wrap(out)

    def matmul(self, sa, la: Layout, sb, lb: Layout, dt: int) -> DeviceStorage:
        out, va, vb = ctypes.c_void_p(), self._view(sa, la, dt), self._view(sb, lb, dt)
        self.check(self.lib.wb_matmul(self.handle, ctypes.byref(va), ctypes.byref(vb), ctypes.byref(out)))
        return self._wrap(out)

    def im2col(self, s, l: Layout, dt: int, p: Im2ColParams) -> DeviceStorage:
        out, v, cp = ctypes.c_void_p(), self._view(s, l, dt), WbConvParams(*p.as_args())
        self.check(self.lib.wb_im2col(self.handle, ctypes.byref(v), ctypes.byref(cp), ctypes.byref(out)))
        return self._wrap(out)

    def col2im(self, s, l: Layout, dt: int, p: Im2ColParams, chw) -> DeviceStorage:
        out, v, cp = ctypes.c_void_p(), self._view(s, l, dt), WbConvParams(*p.as_args())
        self.check(self.lib.wb_col2im(self.handle, ctypes.byref(v), ctypes.byref(cp), *chw, ctypes.byref(out)))
        return self._wrap(out)

    def cast(self, s, l: Layout, dt: int, to: int) -> DeviceStorage:
        out, v = ctypes.c_void_p(), self._view(s, l, dt)
        self.check(self.lib.wb_cast(self.handle, ctypes.byref(v), to, ctypes.byref(out)))
        return self._wrap(out)

    def random(self, n: int, dt: int, dist: Distribution, seed: int) -> DeviceStorage:
        out = ctypes.c_void_p()
        self.check(self.lib.wb_random(self.handle, n, dt, dist.kind, dist.a, dist.b, seed, ctypes.byref(out)))
        return self._wrap(out)


def device_count() -> int:
    """weta_cuda::device_count (crates/weta-cuda/src/lib.rs:149-152)."""
    return load_library().wb_device_count()


def is_available() -> bool:
    return device_count() > 0
