"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: Python binding of the CPU oracle.

`OracleBackend` exposes the restated weta-cpu kernels (oracle/weta_cpu_oracle.cpp, which cites
crates/weta-cpu/src/lib.rs line by line) through the same method set the product's backend
object has, with numpy arrays as storage.  Tests run a computation once on this object and once
on the CUDA backend and compare.  Nothing under `weta_b200/` imports this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

from weta_b200.core import Distribution, DType, Im2ColParams, Layout, WbView

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libweta_cpu_oracle.so")


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "weta_cpu_oracle.cpp")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libweta_cpu_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB


def _load():
    lib = ctypes.CDLL(build())
    P, V = ctypes.c_void_p, ctypes.POINTER(WbView)
    i64, i32, f64, u64 = ctypes.c_int64, ctypes.c_int, ctypes.c_double, ctypes.c_uint64
    lib.wo_unary.argtypes = [i32, f64, f64, V, P]
    lib.wo_binary.argtypes = [i32, V, V, P]
    lib.wo_reduce.argtypes = [i32, V, i32, P]
    lib.wo_matmul.argtypes = [V, V, P]
    lib.wo_im2col.argtypes = [V] + [i64] * 8 + [P]
    lib.wo_col2im.argtypes = [V] + [i64] * 11 + [P]
    lib.wo_copy_strided.argtypes = [V, V]
    lib.wo_cast.argtypes = [V, i32, P]
    lib.wo_random.argtypes = [i64, i32, i32, f64, f64, u64, P]
    lib.wo_splitmix64.argtypes = [u64, u64]
    lib.wo_splitmix64.restype = u64
    lib.wo_set_num_threads.argtypes = [i32]
    lib.wo_set_matmul_test_mode.argtypes = [i32, i32]
    return lib


class OracleBackend:
    """weta-cpu restated; storage is a 1-D numpy array."""

    name = "oracle-cpu"

    def __init__(self):
        self.lib = _load()

    def num_threads(self) -> int:
        return int(self.lib.wo_num_threads())

    def set_num_threads(self, n: int) -> None:
        self.lib.wo_set_num_threads(int(n))

    def set_matmul_test_mode(self, tf32_operands: int = 0, f64_accumulate: bool = False) -> None:
        """f32 matmul with operands reduced to TF32 (0 off, 1 low 13 mantissa bits dropped, 2 rounded to nearest with ties
        away from zero, 3 rounded to nearest even) and / or the sum over k kept in double; both off restores the plain
        restatement of weta-cpu."""
        self.lib.wo_set_matmul_test_mode(int(tf32_operands), int(f64_accumulate))

    # helpers
    @staticmethod
    def _view(s: np.ndarray, l: Layout, dt: int) -> WbView:
        return l.view(s.ctypes.data, dt)

    @staticmethod
    def _out(n: int, dt: int) -> np.ndarray:
        return np.empty(max(n, 1), dtype=DType.np(dt))[:n] if n else np.empty(0, dtype=DType.np(dt))

    def _check(self, rc: int, what: str):
        if rc != 0:
            raise RuntimeError(f"oracle {what}: unsupported dtype or op (code {rc})")

    # trait surface (crates/weta-core/src/backend.rs:65-106)
    def from_host(self, flat: np.ndarray) -> np.ndarray:
        return np.array(flat, copy=True).reshape(-1)

    def to_host(self, s, l: Layout, dt: int) -> np.ndarray:
        out = self._out(l.numel(), dt)
        self._check(self.lib.wo_cast(self._view(s, l, dt), dt, out.ctypes.data), "to_host")
        return out

    def zeros(self, n: int, dt: int) -> np.ndarray:
        return np.zeros(n, dtype=DType.np(dt))

    def copy_strided(self, src, ls: Layout, dt: int, dst, ld: Layout) -> None:
        self._check(self.lib.wo_copy_strided(self._view(src, ls, dt), self._view(dst, ld, dt)), "copy_strided")

    def unary(self, op: int, p1: float, p2: float, s, l: Layout, dt: int):
        out = self._out(l.numel(), dt)
        self._check(self.lib.wo_unary(op, p1, p2, self._view(s, l, dt), out.ctypes.data), "unary")
        return out

    def binary(self, op: int, sa, la: Layout, sb, lb: Layout, dt: int):
        out = self._out(la.numel(), dt)
        self._check(self.lib.wo_binary(op, self._view(sa, la, dt), self._view(sb, lb, dt), out.ctypes.data), "binary")
        return out

    def reduce(self, op: int, s, l: Layout, dt: int, axis: int):
        n_out = l.numel() // max(l.shape[axis], 1) if l.shape[axis] else int(np.prod(
            [d for i, d in enumerate(l.shape) if i != axis], dtype=np.int64))
        out = self._out(n_out, DType.I64 if op >= 3 else dt)
        self._check(self.lib.wo_reduce(op, self._view(s, l, dt), axis, out.ctypes.data), "reduce")
        return out

    def matmul(self, sa, la: Layout, sb, lb: Layout, dt: int):
        out = self._out(la.shape[0] * la.shape[1] * lb.shape[2], dt)
        self._check(self.lib.wo_matmul(self._view(sa, la, dt), self._view(sb, lb, dt), out.ctypes.data), "matmul")
        return out

    def im2col(self, s, l: Layout, dt: int, p: Im2ColParams):
        n, c, h, w = l.shape
        oh, ow = p.out_size(h, w)
        out = self._out(n * c * p.kernel[0] * p.kernel[1] * oh * ow, dt)
        self._check(self.lib.wo_im2col(self._view(s, l, dt), *p.as_args(), out.ctypes.data), "im2col")
        return out

    def col2im(self, s, l: Layout, dt: int, p: Im2ColParams, chw):
        out = self._out(l.shape[0] * chw[0] * chw[1] * chw[2], dt)
        self._check(self.lib.wo_col2im(self._view(s, l, dt), *p.as_args(), *chw, out.ctypes.data), "col2im")
        return out

    def cast(self, s, l: Layout, dt: int, to: int):
        out = self._out(l.numel(), to)
        self._check(self.lib.wo_cast(self._view(s, l, dt), to, out.ctypes.data), "cast")
        return out

    def random(self, n: int, dt: int, dist: Distribution, seed: int):
        out = self._out(n, dt)
        self._check(self.lib.wo_random(n, dt, dist.kind, dist.a, dist.b, seed, out.ctypes.data), "random")
        return out

    def synchronize(self) -> None:
        pass
