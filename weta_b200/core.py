"""Vocabulary shared by every layer above the C ABI: dtypes, op codes, layouts, the host RNG.

Mirrors `weta-core` (crates/weta-core/src/{dtype,ops,layout}.rs) and the global seed stream
of `weta-tensor` (crates/weta-tensor/src/random.rs:21-110).  Op codes are the ones the
reference CUDA backend passes to its kernels (crates/weta-cuda/src/lib.rs:256-296), so a
binding written against that numbering keeps working.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

MAX_DIMS = 8  # crates/weta-cuda/src/lib.rs:67


class DType:
    """crates/weta-core/src/dtype.rs:9-22"""

    F32, F64, I64 = 0, 1, 2
    _np = {0: np.float32, 1: np.float64, 2: np.int64}
    _size = {0: 4, 1: 8, 2: 8}
    _name = {0: "f32", 1: "f64", 2: "i64"}

    @staticmethod
    def np(dt: int):
        return DType._np[dt]

    @staticmethod
    def size(dt: int) -> int:
        return DType._size[dt]

    @staticmethod
    def name(dt: int) -> str:
        return DType._name[dt]

    @staticmethod
    def of(arr: np.ndarray) -> int:
        for k, v in DType._np.items():
            if arr.dtype == v:
                return k
        raise TypeError(f"unsupported dtype {arr.dtype}")

    @staticmethod
    def is_float(dt: int) -> bool:
        return dt in (0, 1)


class UnaryOp:
    """crates/weta-core/src/ops.rs:7-36; codes from crates/weta-cuda/src/lib.rs:256-278"""

    NEG, EXP, LOG, SQRT, ABS, SIGN, RELU, STEP, TANH, SIGMOID, ERF, SIN, COS, RECIP = range(14)
    AFFINE, POWF, GT_SCALAR, MAX_SCALAR, MIN_SCALAR = 14, 15, 16, 17, 18
    NAMES = ["neg", "exp", "log", "sqrt", "abs", "sign", "relu", "step", "tanh", "sigmoid", "erf", "sin", "cos",
             "reciprocal", "affine", "pow", "gt", "clamp_min", "clamp_max"]
    INT_OK = (0, 4, 5, 6, 7, 14, 16, 17, 18)  # crates/weta-cpu/src/lib.rs:190-203


class BinaryOp:
    """crates/weta-core/src/ops.rs:68-82; codes from crates/weta-cuda/src/lib.rs:280-296"""

    ADD, SUB, MUL, DIV, POW, MAXIMUM, MINIMUM, EQ, NE, LT, LE, GT, GE = range(13)
    NAMES = ["add", "sub", "mul", "div", "pow", "maximum", "minimum", "eq", "ne", "lt", "le", "gt", "ge"]


class ReduceOp:
    """crates/weta-core/src/ops.rs:106-112"""

    SUM, MAX, MIN, ARGMAX, ARGMIN = range(5)


@dataclass(frozen=True)
class Im2ColParams:
    """crates/weta-core/src/ops.rs:122-150"""

    kernel: Tuple[int, int]
    stride: Tuple[int, int] = (1, 1)
    padding: Tuple[int, int] = (0, 0)
    dilation: Tuple[int, int] = (1, 1)

    def out_size(self, h: int, w: int) -> Tuple[int, int]:
        def f(x, k, s, p, d):
            span = d * (k - 1) + 1
            return 0 if x + 2 * p < span else (x + 2 * p - span) // s + 1

        return (f(h, self.kernel[0], self.stride[0], self.padding[0], self.dilation[0]),
                f(w, self.kernel[1], self.stride[1], self.padding[1], self.dilation[1]))

    def as_args(self):
        return (*self.kernel, *self.stride, *self.padding, *self.dilation)


@dataclass(frozen=True)
class Distribution:
    """crates/weta-core/src/ops.rs:154-157.  kind 0 = Uniform{lo,hi}, 1 = Normal{mean,std}."""

    kind: int
    a: float
    b: float

    @staticmethod
    def uniform(lo: float, hi: float) -> "Distribution":
        return Distribution(0, lo, hi)

    @staticmethod
    def normal(mean: float, std: float) -> "Distribution":
        return Distribution(1, mean, std)


class WbView(ctypes.Structure):
    """The strided view every op takes (include/weta_b200.h `WbView`): a storage base pointer,
    dtype, rank, and shape / stride / offset counted in elements."""

    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("ndim", ctypes.c_int32),
                ("shape", ctypes.c_int64 * MAX_DIMS), ("stride", ctypes.c_int64 * MAX_DIMS),
                ("offset", ctypes.c_int64)]


def contiguous_strides(shape: Sequence[int]) -> List[int]:
    strides = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        strides[i] = strides[i + 1] * max(shape[i + 1], 1)
    return strides


class Layout:
    """crates/weta-core/src/layout.rs:16-21: shape, strides and offset, all in elements."""

    __slots__ = ("shape", "strides", "offset")

    def __init__(self, shape: Sequence[int], strides: Sequence[int], offset: int = 0):
        assert len(shape) == len(strides)
        self.shape = tuple(int(s) for s in shape)
        self.strides = tuple(int(s) for s in strides)
        self.offset = int(offset)

    @staticmethod
    def contiguous(shape: Sequence[int]) -> "Layout":
        return Layout(shape, contiguous_strides(shape), 0)

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def numel(self) -> int:
        return math.prod(self.shape)

    def is_contiguous(self) -> bool:  # layout.rs:60-69
        expected = 1
        for d, s in zip(reversed(self.shape), reversed(self.strides)):
            if d != 1 and s != expected:
                return False
            expected *= d
        return True

    def transpose(self, d0: int, d1: int) -> "Layout":
        sh, st = list(self.shape), list(self.strides)
        sh[d0], sh[d1] = sh[d1], sh[d0]
        st[d0], st[d1] = st[d1], st[d0]
        return Layout(sh, st, self.offset)

    def permute(self, dims: Sequence[int]) -> "Layout":
        assert sorted(dims) == list(range(self.ndim)), f"{dims} is not a permutation of {self.ndim} dims"
        return Layout([self.shape[d] for d in dims], [self.strides[d] for d in dims], self.offset)

    def narrow(self, dim: int, start: int, length: int) -> "Layout":
        assert dim < self.ndim and start + length <= self.shape[dim]
        sh = list(self.shape)
        sh[dim] = length
        return Layout(sh, self.strides, self.offset + start * self.strides[dim])

    def step(self, dim: int, step: int) -> "Layout":  # layout.rs:115-120
        sh, st = list(self.shape), list(self.strides)
        sh[dim] = -(-sh[dim] // step)
        st[dim] *= step
        return Layout(sh, st, self.offset)

    def unsqueeze(self, dim: int) -> "Layout":  # layout.rs:122-131
        sh, st = list(self.shape), list(self.strides)
        stride = st[dim] * sh[dim] if dim < self.ndim else 1
        sh.insert(dim, 1)
        st.insert(dim, stride)
        return Layout(sh, st, self.offset)

    def squeeze(self, dim: int) -> "Layout":
        assert self.shape[dim] == 1
        sh, st = list(self.shape), list(self.strides)
        del sh[dim], st[dim]
        return Layout(sh, st, self.offset)

    def broadcast_to(self, shape: Sequence[int]) -> "Layout":  # layout.rs:146-161
        assert len(shape) >= self.ndim, f"can't broadcast {self.shape} to {tuple(shape)}"
        extra = len(shape) - self.ndim
        strides = [0] * len(shape)
        for i in range(extra, len(shape)):
            d = self.shape[i - extra]
            if d == shape[i]:
                strides[i] = self.strides[i - extra]
            elif d != 1:
                raise ValueError(f"can't broadcast {self.shape} to {tuple(shape)}")
        return Layout(shape, strides, self.offset)

    def reshape(self, shape: Sequence[int]) -> Optional["Layout"]:  # layout.rs:165-171
        if self.is_contiguous():
            return Layout(shape, contiguous_strides(shape), self.offset)
        return None

    def offsets(self) -> np.ndarray:
        """Storage index of every element in row-major order (layout.rs:226-263)."""
        off = np.full((), self.offset, dtype=np.int64)
        for d, s in zip(self.shape, self.strides):
            off = off[..., None] + np.arange(d, dtype=np.int64) * s
        return off.reshape(-1)

    def view(self, data: int, dtype: int) -> WbView:
        assert self.ndim <= MAX_DIMS, f"at most {MAX_DIMS} dims are supported, got shape {self.shape}"
        v = WbView()
        v.data = data
        v.dtype = dtype
        v.ndim = self.ndim
        for i in range(MAX_DIMS):
            v.shape[i] = self.shape[i] if i < self.ndim else 1
            v.stride[i] = self.strides[i] if i < self.ndim else 0
        v.offset = self.offset
        return v

    def __repr__(self):
        return f"Layout(shape={self.shape}, strides={self.strides}, offset={self.offset})"


def resolve_shape(numel: int, shape: Sequence[int]) -> List[int]:
    """crates/weta-core/src/layout.rs:180-205: resolves one -1."""
    shape = list(shape)
    if shape.count(-1) > 1:
        raise ValueError("only one dimension can be -1")
    if -1 in shape:
        known = math.prod(s for s in shape if s != -1)
        if known == 0 or numel % known:
            raise ValueError(f"can't reshape {numel} elements to {shape}")
        shape[shape.index(-1)] = numel // known
    if math.prod(shape) != numel:
        raise ValueError(f"can't reshape {numel} elements to {shape}")
    return shape


def broadcast_shapes(a: Sequence[int], b: Sequence[int]) -> List[int]:
    """crates/weta-core/src/layout.rs:207-224"""
    n = max(len(a), len(b))
    out = []
    for i in range(n):
        da = a[len(a) - n + i] if len(a) - n + i >= 0 else 1
        db = b[len(b) - n + i] if len(b) - n + i >= 0 else 1
        if da == db or db == 1:
            out.append(da)
        elif da == 1:
            out.append(db)
        else:
            raise ValueError(f"shapes {tuple(a)} and {tuple(b)} don't broadcast")
    return out


_M64 = (1 << 64) - 1


def splitmix64(seed: int, i: int) -> int:
    """crates/weta-core/src/ops.rs:164-169"""
    z = (seed + ((i + 1) * 0x9E3779B97F4A7C15)) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


class Pcg:
    """PCG-XSH-RR, the host generator that hands one 64-bit seed to each random tensor
    (crates/weta-tensor/src/random.rs:21-74)."""

    INC = ((0xDA3E39CB94B95BDB << 1) | 1) & _M64
    MUL = 6364136223846793005
    DEFAULT_SEED = 67280421310721  # random.rs:77

    def __init__(self, seed: int):
        self.state = 0
        self.next_u32()
        self.state = (self.state + seed) & _M64
        self.next_u32()

    def next_u32(self) -> int:
        old = self.state
        self.state = (old * self.MUL + self.INC) & _M64
        xorshifted = (((old >> 18) ^ old) >> 27) & 0xFFFFFFFF
        rot = old >> 59
        return ((xorshifted >> rot) | (xorshifted << ((-rot) & 31))) & 0xFFFFFFFF

    def next_u64(self) -> int:
        hi = self.next_u32()
        return (hi << 32) | self.next_u32()

    def uniform(self) -> float:
        hi = self.next_u32() >> 5
        lo = self.next_u32() >> 6
        return ((hi << 26) | lo) / float(1 << 53)

    def below(self, n: int) -> int:
        return int(self.uniform() * n) % max(n, 1)


_global_rng: Optional[Pcg] = None


def manual_seed(seed: int) -> None:
    """crates/weta-tensor/src/random.rs:88-90"""
    global _global_rng
    _global_rng = Pcg(seed)


def global_rng() -> Pcg:
    global _global_rng
    if _global_rng is None:
        _global_rng = Pcg(Pcg.DEFAULT_SEED)
    return _global_rng
