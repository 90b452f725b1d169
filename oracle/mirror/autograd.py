"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: reverse-mode autograd over `Tensor`, emitting the primitive sequences of `weta-autograd`.

Each backward rule below issues the tensor ops of the corresponding rule in
crates/weta-autograd/src/ops.rs (cited per rule), visited in reverse creation order like
crates/weta-autograd/src/graph.rs:227-276.  The point is not a general framework: it lets the
named models' training step run "in primitive mode" on any backend object, producing the same
~400 backend calls per step the reference produces, for parity and for baseline timing.
"""
from __future__ import annotations

import itertools
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np

from weta_b200.core import BinaryOp, DType, Im2ColParams, UnaryOp
from .tensor import Tensor

_seq = itertools.count()
_grad_enabled = True


class no_grad:
    def __enter__(self):
        global _grad_enabled
        self.prev, _grad_enabled = _grad_enabled, False

    def __exit__(self, *a):
        global _grad_enabled
        _grad_enabled = self.prev


class Node:
    __slots__ = ("seq", "name", "backward", "inputs", "in_shapes", "needs")

    def __init__(self, name: str, backward: Callable, inputs: Sequence["Var"]):
        self.seq = next(_seq)
        self.name = name
        self.backward = backward
        self.inputs = list(inputs)
        self.in_shapes = [tuple(v.shape) for v in inputs]
        self.needs = [v.requires_grad or v.node is not None for v in inputs]


class Var:
    """An autograd tensor: raw data, an optional producing node, an optional leaf gradient."""

    def __init__(self, data: Tensor, requires_grad: bool = False, node: Optional[Node] = None):
        self.data = data
        self.requires_grad = requires_grad
        self.node = node
        self.grad: Optional[Tensor] = None

    # -- plumbing ---------------------------------------------------------------------------
    @property
    def shape(self):
        return self.data.shape

    @property
    def ndim(self):
        return self.data.ndim

    @property
    def dtype(self):
        return self.data.dtype

    def size(self, d):
        return self.data.size(d)

    def numel(self):
        return self.data.numel()

    def detach(self) -> "Var":
        return Var(self.data)

    def item(self) -> float:
        return self.data.item()

    def numpy(self) -> np.ndarray:
        return self.data.numpy()

    @staticmethod
    def _from_op(out: Tensor, name: str, inputs: Sequence["Var"], backward: Callable) -> "Var":
        if _grad_enabled and any(v.requires_grad or v.node is not None for v in inputs):
            return Var(out, node=Node(name, backward, inputs))
        return Var(out)

    def backward(self, grad: Optional[Tensor] = None) -> None:
        """crates/weta-autograd/src/graph.rs:227-276"""
        if grad is None:
            assert self.numel() == 1, "grad can be implicitly created only for scalar outputs"
            grad = Tensor.full(self.shape, 1.0, self.dtype, self.data.backend)
        if self.node is None:
            if self.requires_grad:
                self._accumulate(grad)
            return
        nodes, seen, stack = [], {id(self.node)}, [self.node]
        while stack:
            n = stack.pop()
            nodes.append(n)
            for v in n.inputs:
                if v.node is not None and id(v.node) not in seen:
                    seen.add(id(v.node))
                    stack.append(v.node)
        nodes.sort(key=lambda n: -n.seq)
        grads = {id(self.node): grad}
        with no_grad():
            for n in nodes:
                g = grads.pop(id(n), None)
                if g is None:
                    continue
                for v, gi, want in zip(n.inputs, n.backward(n, g), n.in_shapes):
                    if gi is None:
                        continue
                    assert tuple(gi.shape) == want, f"{n.name}: gradient shape {gi.shape}, expected {want}"
                    if v.node is not None:
                        prev = grads.get(id(v.node))
                        grads[id(v.node)] = gi if prev is None else prev.add(gi)
                    elif v.requires_grad:
                        v._accumulate(gi)

    def _accumulate(self, g: Tensor) -> None:
        self.grad = g if self.grad is None else self.grad.add(g)

    # -- element-wise unary (ops.rs:64-108) -------------------------------------------------
    def unary(self, op: int, p1: float = 0.0, p2: float = 0.0) -> "Var":
        x = self.data

        def bw(n: Node, g: Tensor):
            U = UnaryOp
            if op == U.NEG: gx = g.neg()
            elif op == U.EXP: gx = g.mul(x.exp())
            elif op == U.LOG: gx = g.div(x)
            elif op == U.SQRT: gx = g.mul(x.sqrt().reciprocal()).mul_scalar(0.5)
            elif op == U.ABS: gx = g.mul(x.sign())
            elif op in (U.SIGN, U.STEP, U.GT_SCALAR): gx = Tensor.zeros(g.shape, g.dtype, g.backend)
            elif op == U.RELU: gx = g.mul(x.step())
            elif op == U.TANH:
                t = x.tanh()
                gx = g.mul(t.mul(t).affine(-1.0, 1.0))
            elif op == U.SIGMOID:
                s = x.sigmoid()
                gx = g.mul(s.mul(s.affine(-1.0, 1.0)))
            elif op == U.ERF: gx = g.mul(x.mul(x).neg().exp()).mul_scalar(1.1283791670955126)
            elif op == U.SIN: gx = g.mul(x.cos())
            elif op == U.COS: gx = g.mul(x.sin()).neg()
            elif op == U.RECIP: gx = g.div(x.mul(x)).neg()
            elif op == U.AFFINE: gx = g.mul_scalar(p1)
            elif op == U.POWF: gx = g.mul(x.powf(p1 - 1.0)).mul_scalar(p1)
            elif op == U.MAX_SCALAR: gx = g.mul(x.gt_scalar(p1))
            elif op == U.MIN_SCALAR: gx = g.mul(x.neg().gt_scalar(-p1))
            else: raise ValueError(op)
            return [gx]

        return Var._from_op(x.unary(op, p1, p2), UnaryOp.NAMES[op], [self], bw)

    def relu(self): return self.unary(UnaryOp.RELU)
    def exp(self): return self.unary(UnaryOp.EXP)
    def log(self): return self.unary(UnaryOp.LOG)
    def sqrt(self): return self.unary(UnaryOp.SQRT)
    def tanh(self): return self.unary(UnaryOp.TANH)
    def sigmoid(self): return self.unary(UnaryOp.SIGMOID)
    def erf(self): return self.unary(UnaryOp.ERF)
    def reciprocal(self): return self.unary(UnaryOp.RECIP)
    def neg(self): return self.unary(UnaryOp.NEG)
    def affine(self, mul, add): return self.unary(UnaryOp.AFFINE, mul, add)
    def mul_scalar(self, v): return self.affine(v, 0.0)      # `t * s`   (ops.rs:1026)
    def add_scalar(self, v): return self.affine(1.0, v)      # `t + s`   (ops.rs:1024)

    # -- element-wise binary with broadcasting (ops.rs:183-220) -----------------------------
    def binary(self, op: int, other: "Var") -> "Var":
        a, b = self.data, other.data
        out = a.binary(op, b)
        if op >= BinaryOp.EQ:
            return Var(out)

        def bw(n: Node, g: Tensor):
            B = BinaryOp
            if op == B.ADD: ga, gb = g, g
            elif op == B.SUB: ga, gb = g, g.neg()
            elif op == B.MUL: ga, gb = g.mul(b), g.mul(a)          # both products, eagerly
            elif op == B.DIV: ga, gb = g.div(b), g.mul(a).div(b.mul(b)).neg()
            elif op == B.POW:
                p = a.pow(b)
                ga, gb = g.mul(b).mul(a.pow(b.add_scalar(-1.0))), g.mul(p).mul(a.log())
            else:  # Maximum / Minimum: ties split evenly
                wins, ties = (a.gt(b), a.eq(b)) if op == B.MAXIMUM else (a.lt(b), a.eq(b))
                ma = wins.add(ties.mul_scalar(0.5))
                ga, gb = g.mul(ma), g.mul(ma.affine(-1.0, 1.0))
            return [sum_to_shape(ga, n.in_shapes[0]) if n.needs[0] else None,
                    sum_to_shape(gb, n.in_shapes[1]) if n.needs[1] else None]

        return Var._from_op(out, BinaryOp.NAMES[op], [self, other], bw)

    def add(self, o): return self.binary(BinaryOp.ADD, o)
    def sub(self, o): return self.binary(BinaryOp.SUB, o)
    def mul(self, o): return self.binary(BinaryOp.MUL, o)
    def div(self, o): return self.binary(BinaryOp.DIV, o)

    # -- reductions (ops.rs:274-383) --------------------------------------------------------
    def _norm_dims(self, dims) -> List[int]:
        return sorted({self.data.dim_index(d) for d in dims})

    def sum_dims(self, dims, keepdim=False) -> "Var":
        nd = self._norm_dims(dims)

        def bw(n: Node, g: Tensor):
            shape = n.in_shapes[0]
            return [_unsqueeze_dims(g, shape, nd, keepdim).broadcast_to(shape)]

        return Var._from_op(self.data.sum_dims(dims, keepdim), "sum", [self], bw)

    def sum(self): return self.sum_dims(list(range(self.ndim)), False)

    def mean_dims(self, dims, keepdim=False) -> "Var":
        n = int(np.prod([self.shape[d] for d in self._norm_dims(dims)], dtype=np.int64))
        return self.sum_dims(dims, keepdim).mul_scalar(1.0 / n)

    def mean(self): return self.sum().mul_scalar(1.0 / self.numel())

    def max_dims(self, dims, keepdim=False) -> "Var":
        nd, x = self._norm_dims(dims), self.data
        out = x.max_dims(dims, keepdim)

        def bw(n: Node, g: Tensor):  # MaxBw, ops.rs:305-314
            shape = n.in_shapes[0]
            m = _unsqueeze_dims(out, shape, nd, keepdim)
            mask = x.eq(m).to_dtype(x.dtype)
            count = mask.sum_dims(nd, True)
            return [mask.div(count).mul(_unsqueeze_dims(g, shape, nd, keepdim))]

        return Var._from_op(out, "max", [self], bw)

    def var_dims(self, dims, unbiased: bool, keepdim: bool) -> "Var":  # ops.rs:378-383
        n = int(np.prod([self.shape[d] for d in self._norm_dims(dims)], dtype=np.int64))
        c = self.sub(self.mean_dims(dims, True))
        denom = max(n - 1, 1) if unbiased else n
        return c.mul(c).sum_dims(dims, keepdim).mul_scalar(1.0 / denom)

    def logsumexp(self, dim: int, keepdim: bool) -> "Var":  # ops.rs:386-394
        m = self.max_dims([dim], True).detach()
        out = self.sub(m).exp().sum_dims([dim], True).log().add(m)
        return out if keepdim else out.squeeze(dim)

    def softmax(self, dim: int) -> "Var":  # ops.rs:401-418
        s = self.data.softmax(dim)

        def bw(n: Node, g: Tensor):
            dot = s.mul(g).sum_dims([dim], True)
            return [s.mul(g.sub(dot))]

        return Var._from_op(s, "softmax", [self], bw)

    def log_softmax(self, dim: int) -> "Var":  # ops.rs:420-435
        out = self.data.log_softmax(dim)

        def bw(n: Node, g: Tensor):
            return [g.sub(out.exp().mul(g.sum_dims([dim], True)))]

        return Var._from_op(out, "log_softmax", [self], bw)

    def cross_entropy(self, target: Tensor, reduction: str = "mean", label_smoothing: float = 0.0) -> "Var":
        """crates/weta-autograd/src/ops.rs:444-519; `target` holds I64 class indices [N]."""
        assert self.ndim == 2 and target.dtype == DType.I64 and tuple(target.shape) == (self.shape[0],)
        z = self.data
        c = z.shape[1]
        lsm = z.log_softmax(1)
        y = _smoothed_targets(target, c, label_smoothing, z.dtype)
        per_sample = lsm.mul(y).sum_dims([1], False).neg()
        out = {"none": lambda: per_sample, "mean": per_sample.mean, "sum": per_sample.sum}[reduction]()
        probs = lsm.exp()

        def bw(n: Node, g: Tensor):
            nrows = probs.shape[0]
            diff = probs.sub(_smoothed_targets(target, c, label_smoothing, probs.dtype))
            if reduction == "mean":
                gx = diff.mul(g.mul_scalar(1.0 / nrows))
            elif reduction == "sum":
                gx = diff.mul(g)
            else:
                gx = diff.mul(g.unsqueeze(1))
            return [gx]

        return Var._from_op(out, "cross_entropy", [self], bw)

    # -- views (ops.rs:526-620) -------------------------------------------------------------
    def reshape(self, shape) -> "Var":
        return Var._from_op(self.data.reshape(shape), "reshape", [self],
                            lambda n, g: [g.reshape(list(n.in_shapes[0]))])

    def flatten(self, start=0, end=-1) -> "Var":
        return Var._from_op(self.data.flatten(start, end), "reshape", [self],
                            lambda n, g: [g.reshape(list(n.in_shapes[0]))])

    def squeeze(self, dim) -> "Var":
        return Var._from_op(self.data.squeeze(dim), "reshape", [self], lambda n, g: [g.reshape(list(n.in_shapes[0]))])

    def unsqueeze(self, dim) -> "Var":
        return Var._from_op(self.data.unsqueeze(dim), "reshape", [self], lambda n, g: [g.reshape(list(n.in_shapes[0]))])

    def permute(self, dims) -> "Var":
        inv = [0] * len(dims)
        for i, d in enumerate(dims):
            inv[d] = i
        return Var._from_op(self.data.permute(dims), "permute", [self], lambda n, g: [g.permute(inv)])

    def transpose(self, d0, d1) -> "Var":
        dims = list(range(self.ndim))
        a, b = self.data.dim_index(d0), self.data.dim_index(d1)
        dims[a], dims[b] = dims[b], dims[a]
        return self.permute(dims)

    def t(self) -> "Var":
        return self.transpose(-2, -1)

    # -- matmul / im2col (ops.rs:810-882) ---------------------------------------------------
    def matmul(self, other: "Var") -> "Var":
        if self.ndim == 1 and other.ndim >= 1:
            return self.unsqueeze(0).matmul(other).squeeze(-2)
        if other.ndim == 1 and self.ndim >= 2:
            return self.matmul(other.unsqueeze(1)).squeeze(-1)
        a, b = self.data, other.data

        def bw(n: Node, g: Tensor):
            return [sum_to_shape(g.matmul(b.t()), n.in_shapes[0]) if n.needs[0] else None,
                    sum_to_shape(a.t().matmul(g), n.in_shapes[1]) if n.needs[1] else None]

        return Var._from_op(a.matmul(b), "matmul", [self, other], bw)

    def im2col(self, p: Im2ColParams) -> "Var":
        def bw(n: Node, g: Tensor):
            s = n.in_shapes[0]
            return [g.col2im(p, (s[1], s[2], s[3]))]

        return Var._from_op(self.data.im2col(p), "im2col", [self], bw)


def _unsqueeze_dims(g: Tensor, in_shape, dims, keepdim: bool) -> Tensor:  # ops.rs:259-268
    if keepdim:
        return g
    shape = list(in_shape)
    for d in dims:
        shape[d] = 1
    return g.reshape(shape)


def sum_to_shape(g: Tensor, shape) -> Tensor:  # ops.rs:46-58
    if tuple(g.shape) == tuple(shape):
        return g
    extra = g.ndim - len(shape)
    dims = list(range(extra))
    for i, d in enumerate(shape):
        if d == 1 and g.shape[extra + i] != 1:
            dims.append(extra + i)
    return g.sum_dims(dims, True).reshape(list(shape))


def _smoothed_targets(target: Tensor, classes: int, smoothing: float, dtype: int) -> Tensor:  # ops.rs:472-479
    y = target.one_hot(classes, dtype)
    return y.affine(1.0 - smoothing, smoothing / classes) if smoothing > 0.0 else y
