"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: a strided tensor over a backend object, with the composite ops of `weta-tensor`.

This is the call-site mirror of crates/weta-tensor/src/tensor.rs: every method issues the same
sequence of backend primitives the reference issues (one `reduce` per axis, highest axis first;
softmax as max/sub/exp/sum/div; conv2d as im2col + matmul + add; ...), so a backend plugged in
underneath sees the same traffic as `weta_core::Backend` does.  The class is generic over the
backend object; it never names a concrete one.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np

from weta_b200.core import (BinaryOp, Distribution, DType, Im2ColParams, Layout, ReduceOp, UnaryOp, broadcast_shapes,
                   global_rng, resolve_shape)


class Tensor:
    """Storage handle + layout + dtype + backend.  Views share the storage."""

    __slots__ = ("storage", "layout", "dtype", "backend")

    def __init__(self, storage, layout: Layout, dtype: int, backend):
        self.storage = storage
        self.layout = layout
        self.dtype = dtype
        self.backend = backend

    # -- construction -----------------------------------------------------------------------
    @staticmethod
    def from_numpy(arr: np.ndarray, backend) -> "Tensor":
        arr = np.asarray(arr)
        shape = arr.shape  # np.ascontiguousarray would turn a 0-d array into 1-d
        dt = DType.of(arr)
        return Tensor(backend.from_host(np.ascontiguousarray(arr).reshape(-1)), Layout.contiguous(shape), dt, backend)

    @staticmethod
    def scalar(v: float, dtype: int, backend) -> "Tensor":
        return Tensor.from_numpy(np.array(v, dtype=DType.np(dtype)), backend)

    @staticmethod
    def zeros(shape: Sequence[int], dtype: int, backend) -> "Tensor":
        l = Layout.contiguous(shape)
        return Tensor(backend.zeros(l.numel(), dtype), l, dtype, backend)

    @staticmethod
    def full(shape: Sequence[int], value: float, dtype: int, backend) -> "Tensor":
        # tensor.rs:130-132: a scalar broadcast then copied
        return Tensor.scalar(value, dtype, backend).broadcast_to(shape).copy()

    @staticmethod
    def ones(shape, dtype, backend) -> "Tensor":
        return Tensor.full(shape, 1.0, dtype, backend)

    @staticmethod
    def arange(start: float, end: float, step: float, dtype: int, backend) -> "Tensor":
        # tensor.rs:143-147: built on the host, cast, uploaded
        n = max(0, int(np.ceil((end - start) / step)))
        v = (start + step * np.arange(n, dtype=np.float64)).astype(DType.np(dtype))
        return Tensor.from_numpy(v, backend)

    @staticmethod
    def random_seeded(shape, dist: Distribution, dtype: int, backend, seed: int) -> "Tensor":
        # random.rs:104-110: integer tensors are drawn as f64 and cast
        l = Layout.contiguous(shape)
        fl = dtype if DType.is_float(dtype) else DType.F64
        t = Tensor(backend.random(l.numel(), fl, dist, seed), l, fl, backend)
        return t.to_dtype(dtype)

    @staticmethod
    def random(shape, dist: Distribution, dtype: int, backend) -> "Tensor":
        # random.rs:95-98: one 64-bit seed from the global generator per tensor
        return Tensor.random_seeded(shape, dist, dtype, backend, global_rng().next_u64())

    @staticmethod
    def rand(shape, dtype, backend) -> "Tensor":
        return Tensor.random(shape, Distribution.uniform(0.0, 1.0), dtype, backend)

    @staticmethod
    def randn(shape, dtype, backend) -> "Tensor":
        return Tensor.random(shape, Distribution.normal(0.0, 1.0), dtype, backend)

    @staticmethod
    def uniform(shape, lo, hi, dtype, backend) -> "Tensor":
        return Tensor.random(shape, Distribution.uniform(lo, hi), dtype, backend)

    # -- accessors --------------------------------------------------------------------------
    @property
    def shape(self) -> Tuple[int, ...]:
        return self.layout.shape

    @property
    def ndim(self) -> int:
        return self.layout.ndim

    def numel(self) -> int:
        return self.layout.numel()

    def size(self, dim: int) -> int:
        return self.shape[self.dim_index(dim)]

    def dim_index(self, dim: int) -> int:
        d = dim + self.ndim if dim < 0 else dim
        assert 0 <= d < max(self.ndim, 1), f"dim {dim} out of range for shape {self.shape}"
        return d

    def is_contiguous(self) -> bool:
        return self.layout.is_contiguous()

    def view_with(self, layout: Layout) -> "Tensor":
        return Tensor(self.storage, layout, self.dtype, self.backend)

    def numpy(self) -> np.ndarray:
        """Elements in row-major order, shaped like the tensor (`to_host`)."""
        return self.backend.to_host(self.storage, self.layout, self.dtype).reshape(self.shape)

    def item(self) -> float:
        assert self.numel() == 1
        return float(self.numpy().reshape(-1)[0])

    def to_backend(self, backend) -> "Tensor":
        """`Tensor::to(device)`: a host round trip (tensor.rs:235-240)."""
        if backend is self.backend:
            return self
        return Tensor.from_numpy(self.numpy(), backend)

    def to_dtype(self, dtype: int) -> "Tensor":
        if dtype == self.dtype:
            return self
        s = self.backend.cast(self.storage, self.layout, self.dtype, dtype)
        return Tensor(s, Layout.contiguous(self.shape), dtype, self.backend)

    def contiguous(self) -> "Tensor":
        return self if self.is_contiguous() else self.copy()

    def copy(self) -> "Tensor":  # tensor.rs:259-262: a same-dtype cast
        s = self.backend.cast(self.storage, self.layout, self.dtype, self.dtype)
        return Tensor(s, Layout.contiguous(self.shape), self.dtype, self.backend)

    # -- views ------------------------------------------------------------------------------
    def reshape(self, shape: Sequence[int]) -> "Tensor":
        shape = resolve_shape(self.numel(), shape)
        l = self.layout.reshape(shape)
        if l is not None:
            return self.view_with(l)
        return self.copy().view_with(Layout.contiguous(shape))

    def transpose(self, d0: int, d1: int) -> "Tensor":
        return self.view_with(self.layout.transpose(self.dim_index(d0), self.dim_index(d1)))

    def t(self) -> "Tensor":
        assert self.ndim >= 2
        return self.transpose(-2, -1)

    def permute(self, dims: Sequence[int]) -> "Tensor":
        return self.view_with(self.layout.permute(dims))

    def narrow(self, dim: int, start: int, length: int) -> "Tensor":
        return self.view_with(self.layout.narrow(self.dim_index(dim), start, length))

    def step_by(self, dim: int, step: int) -> "Tensor":
        return self.view_with(self.layout.step(self.dim_index(dim), step))

    def unsqueeze(self, dim: int) -> "Tensor":
        d = dim + self.ndim + 1 if dim < 0 else dim
        return self.view_with(self.layout.unsqueeze(d))

    def squeeze(self, dim: int) -> "Tensor":
        return self.view_with(self.layout.squeeze(self.dim_index(dim)))

    def flatten(self, start: int = 0, end: int = -1) -> "Tensor":
        s, e = self.dim_index(start), self.dim_index(end)
        shape = list(self.shape[:s]) + [int(np.prod(self.shape[s:e + 1], dtype=np.int64))] + list(self.shape[e + 1:])
        return self.reshape(shape)

    def broadcast_to(self, shape: Sequence[int]) -> "Tensor":
        return self.view_with(self.layout.broadcast_to(shape))

    # -- element-wise -----------------------------------------------------------------------
    def unary(self, op: int, p1: float = 0.0, p2: float = 0.0) -> "Tensor":
        s = self.backend.unary(op, p1, p2, self.storage, self.layout, self.dtype)
        return Tensor(s, Layout.contiguous(self.shape), self.dtype, self.backend)

    def binary(self, op: int, other: "Tensor") -> "Tensor":  # tensor.rs:396-406
        assert self.backend is other.backend, "tensors live on different backends"
        assert self.dtype == other.dtype, f"{BinaryOp.NAMES[op]}: dtype mismatch"
        shape = broadcast_shapes(self.shape, other.shape)
        la, lb = self.layout.broadcast_to(shape), other.layout.broadcast_to(shape)
        s = self.backend.binary(op, self.storage, la, other.storage, lb, self.dtype)
        return Tensor(s, Layout.contiguous(shape), self.dtype, self.backend)

    def affine(self, mul: float, add: float) -> "Tensor":
        return self.unary(UnaryOp.AFFINE, mul, add)

    def add_scalar(self, v): return self.affine(1.0, v)
    def mul_scalar(self, v): return self.affine(v, 0.0)
    def powf(self, e): return self.unary(UnaryOp.POWF, e)
    def gt_scalar(self, v): return self.unary(UnaryOp.GT_SCALAR, v)
    def clamp_min(self, v): return self.unary(UnaryOp.MAX_SCALAR, v)
    def clamp_max(self, v): return self.unary(UnaryOp.MIN_SCALAR, v)
    def neg(self): return self.unary(UnaryOp.NEG)
    def exp(self): return self.unary(UnaryOp.EXP)
    def log(self): return self.unary(UnaryOp.LOG)
    def sqrt(self): return self.unary(UnaryOp.SQRT)
    def abs(self): return self.unary(UnaryOp.ABS)
    def sign(self): return self.unary(UnaryOp.SIGN)
    def relu(self): return self.unary(UnaryOp.RELU)
    def step(self): return self.unary(UnaryOp.STEP)
    def tanh(self): return self.unary(UnaryOp.TANH)
    def sigmoid(self): return self.unary(UnaryOp.SIGMOID)
    def erf(self): return self.unary(UnaryOp.ERF)
    def sin(self): return self.unary(UnaryOp.SIN)
    def cos(self): return self.unary(UnaryOp.COS)
    def reciprocal(self): return self.unary(UnaryOp.RECIP)
    def add(self, o): return self.binary(BinaryOp.ADD, o)
    def sub(self, o): return self.binary(BinaryOp.SUB, o)
    def mul(self, o): return self.binary(BinaryOp.MUL, o)
    def div(self, o): return self.binary(BinaryOp.DIV, o)
    def pow(self, o): return self.binary(BinaryOp.POW, o)
    def maximum(self, o): return self.binary(BinaryOp.MAXIMUM, o)
    def minimum(self, o): return self.binary(BinaryOp.MINIMUM, o)
    def eq(self, o): return self.binary(BinaryOp.EQ, o)
    def ne(self, o): return self.binary(BinaryOp.NE, o)
    def lt(self, o): return self.binary(BinaryOp.LT, o)
    def le(self, o): return self.binary(BinaryOp.LE, o)
    def gt(self, o): return self.binary(BinaryOp.GT, o)
    def ge(self, o): return self.binary(BinaryOp.GE, o)

    # -- reductions (tensor.rs:488-577) -----------------------------------------------------
    def _reduce_axis(self, op: int, axis: int) -> "Tensor":
        s = self.backend.reduce(op, self.storage, self.layout, self.dtype, axis)
        shape = list(self.shape)
        del shape[axis]
        dt = DType.I64 if op in (ReduceOp.ARGMAX, ReduceOp.ARGMIN) else self.dtype
        return Tensor(s, Layout.contiguous(shape), dt, self.backend)

    def _reduce(self, op: int, dims: Sequence[int], keepdim: bool) -> "Tensor":
        axes = sorted({self.dim_index(d) for d in dims})
        out = self
        for a in reversed(axes):  # one backend call per axis, highest axis first
            out = out._reduce_axis(op, a)
        if keepdim:
            for a in axes:
                out = out.unsqueeze(a)
        return out

    def _all_dims(self) -> List[int]:
        return list(range(self.ndim))

    def sum_dims(self, dims, keepdim=False): return self._reduce(ReduceOp.SUM, dims, keepdim)
    def sum(self): return self.sum_dims(self._all_dims(), False)
    def max_dims(self, dims, keepdim=False): return self._reduce(ReduceOp.MAX, dims, keepdim)
    def min_dims(self, dims, keepdim=False): return self._reduce(ReduceOp.MIN, dims, keepdim)
    def max(self): return self.max_dims(self._all_dims(), False)
    def min(self): return self.min_dims(self._all_dims(), False)
    def argmax(self, dim, keepdim=False): return self._reduce(ReduceOp.ARGMAX, [dim], keepdim)
    def argmin(self, dim, keepdim=False): return self._reduce(ReduceOp.ARGMIN, [dim], keepdim)

    def mean_dims(self, dims, keepdim=False) -> "Tensor":
        n = int(np.prod([self.size(d) for d in dims], dtype=np.int64))
        return self.sum_dims(dims, keepdim).mul_scalar(1.0 / n)

    def mean(self) -> "Tensor":
        return self.sum().mul_scalar(1.0 / self.numel())

    def var_dims(self, dims, unbiased: bool, keepdim: bool) -> "Tensor":
        n = int(np.prod([self.size(d) for d in dims], dtype=np.int64))
        centered = self.sub(self.mean_dims(dims, True))
        denom = max(n - 1, 1) if unbiased else n
        return centered.mul(centered).sum_dims(dims, keepdim).mul_scalar(1.0 / denom)

    def logsumexp(self, dim: int, keepdim: bool) -> "Tensor":
        m = self.max_dims([dim], True)
        out = self.sub(m).exp().sum_dims([dim], True).log().add(m)
        return out if keepdim else out.squeeze(dim)

    def softmax(self, dim: int) -> "Tensor":
        e = self.sub(self.max_dims([dim], True)).exp()
        return e.div(e.sum_dims([dim], True))

    def log_softmax(self, dim: int) -> "Tensor":
        return self.sub(self.logsumexp(dim, True))

    # -- matmul / conv (tensor.rs:584-708) --------------------------------------------------
    @staticmethod
    def _merge_batch(l: Layout) -> Optional[Layout]:
        nb = l.ndim - 2
        b, stride, first = 1, 0, True
        for i in range(nb - 1, -1, -1):
            if l.shape[i] == 1:
                continue
            if first:
                stride, first = l.strides[i], False
            elif l.strides[i] != stride * b:
                return None
            b *= l.shape[i]
        return Layout([b, l.shape[nb], l.shape[nb + 1]], [stride, l.strides[nb], l.strides[nb + 1]], l.offset)

    def matmul(self, other: "Tensor") -> "Tensor":
        assert self.dtype == other.dtype and self.ndim >= 1 and other.ndim >= 1
        a = self.unsqueeze(0) if self.ndim == 1 else self
        b = other.unsqueeze(1) if other.ndim == 1 else other
        m, k = a.shape[-2], a.shape[-1]
        k2, n = b.shape[-2], b.shape[-1]
        assert k == k2, f"matmul: {self.shape} x {other.shape}: inner dims {k} != {k2}"
        batch = broadcast_shapes(a.shape[:-2], b.shape[:-2])

        def full(t: Tensor, r: int, c: int) -> Layout:
            l = t.layout.broadcast_to(list(batch) + [r, c])
            return l.unsqueeze(0) if not batch else l

        def merged(t: Tensor, fl: Layout):
            ml = Tensor._merge_batch(fl)
            if ml is not None:
                return t.storage, ml
            c = t.view_with(fl).copy()  # batch dims that don't merge need a copy first
            return c.storage, Tensor._merge_batch(c.layout)

        (sa, la), (sb, lb) = merged(a, full(a, m, k)), merged(b, full(b, k, n))
        s = self.backend.matmul(sa, la, sb, lb, self.dtype)
        shape = list(batch)
        if self.ndim > 1:
            shape.append(m)
        if other.ndim > 1:
            shape.append(n)
        return Tensor(s, Layout.contiguous(shape), self.dtype, self.backend)

    def im2col(self, p: Im2ColParams) -> "Tensor":
        assert self.ndim == 4, f"im2col: expected [N, C, H, W], got {self.shape}"
        n, c, h, w = self.shape
        oh, ow = p.out_size(h, w)
        s = self.backend.im2col(self.storage, self.layout, self.dtype, p)
        return Tensor(s, Layout.contiguous([n, c * p.kernel[0] * p.kernel[1], oh * ow]), self.dtype, self.backend)

    def col2im(self, p: Im2ColParams, chw: Tuple[int, int, int]) -> "Tensor":
        assert self.ndim == 3, f"col2im: expected [N, C*kh*kw, L], got {self.shape}"
        s = self.backend.col2im(self.storage, self.layout, self.dtype, p, chw)
        return Tensor(s, Layout.contiguous([self.shape[0], *chw]), self.dtype, self.backend)

    def conv2d(self, w: "Tensor", b: Optional["Tensor"], stride: int, padding: int) -> "Tensor":
        n, _, h, wd = self.shape
        o, _, kh, kw = w.shape
        p = Im2ColParams((kh, kw), (stride, stride), (padding, padding), (1, 1))
        oh, ow = p.out_size(h, wd)
        out = w.reshape([o, -1]).matmul(self.im2col(p))
        if b is not None:
            out = out.add(b.reshape([o, 1]))
        return out.reshape([n, o, oh, ow])

    def max_pool2d(self, kernel: int, stride: int) -> "Tensor":
        n, c, h, w = self.shape
        p = Im2ColParams((kernel, kernel), (stride, stride))
        oh, ow = p.out_size(h, w)
        cols = self.reshape([n * c, 1, h, w]).im2col(p)
        return cols.max_dims([1], False).reshape([n, c, oh, ow])

    @staticmethod
    def cat(tensors: Sequence["Tensor"], dim: int) -> "Tensor":  # tensor.rs:710-731
        first = tensors[0]
        d = first.dim_index(dim)
        shape = list(first.shape)
        shape[d] = sum(t.shape[d] for t in tensors)
        out = Tensor.zeros(shape, first.dtype, first.backend)
        start = 0
        for t in tensors:
            out.narrow(d, start, t.shape[d]).assign(t)
            start += t.shape[d]
        return out

    def one_hot(self, classes: int, dtype: int) -> "Tensor":  # tensor.rs:747-750
        ids = Tensor.arange(0.0, float(classes), 1.0, DType.I64, self.backend)
        return self.unsqueeze(-1).eq(ids).to_dtype(dtype)

    # -- in place (tensor.rs:762-811) -------------------------------------------------------
    def assign(self, src: "Tensor") -> None:
        src = src.to_backend(self.backend).to_dtype(self.dtype)
        ls = src.layout.broadcast_to(self.shape)
        if src.storage is self.storage:
            tmp = src.view_with(ls).copy()
            self.backend.copy_strided(tmp.storage, tmp.layout, self.dtype, self.storage, self.layout)
        else:
            self.backend.copy_strided(src.storage, ls, self.dtype, self.storage, self.layout)

    def fill_(self, v: float) -> None:
        self.assign(Tensor.scalar(v, self.dtype, self.backend))

    def sub_(self, other: "Tensor") -> None:
        self.assign(self.sub(other))

    def add_(self, other: "Tensor") -> None:
        self.assign(self.add(other))

    def mul_scalar_(self, v: float) -> None:
        self.assign(self.mul_scalar(v))


def allclose(a: np.ndarray, b: np.ndarray, rtol: float, atol: float) -> bool:
    """crates/weta-tensor/src/tensor.rs:814-816: |a - b| <= atol + rtol * |b| (NaN never passes)."""
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return a.shape == b.shape and bool(np.all(np.abs(a - b) <= atol + rtol * np.abs(b)))
