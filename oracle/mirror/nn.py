"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: layers, functional ops, the named models and the optimizers, in primitive mode.

Everything here is written in `Var`/`Tensor` ops in the order the reference writes them
(crates/weta-nn/src/functional.rs, crates/weta-nn/src/layers.rs, crates/weta-optim/src/lib.rs),
so running a model from this module on a backend reproduces the reference's primitive-call
stream: default initialisation order, dropout seeds, BatchNorm bookkeeping, Adam's 13 calls per
parameter.  The fused trainer in `weta_b200.trainer` computes the same step in a few kernels.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

from .autograd import Var, no_grad
from weta_b200.core import DType, Im2ColParams
from .tensor import Tensor


# -- functional (crates/weta-nn/src/functional.rs) -----------------------------------------------
def relu(x: Var) -> Var:
    return x.relu()


def linear(x: Var, weight: Var, bias: Optional[Var]) -> Var:  # :54-60
    y = x.matmul(weight.t())
    return y.add(bias) if bias is not None else y


def dropout(x: Var, p: float, training: bool) -> Var:  # :64-74
    assert 0.0 <= p <= 1.0
    if not training or p == 0.0:
        return x
    if p == 1.0:
        return x.mul_scalar(0.0)
    mask = Tensor.rand(x.shape, x.dtype, x.data.backend).gt_scalar(p).mul_scalar(1.0 / (1.0 - p))
    return x.mul(Var(mask))


def conv2d(x: Var, weight: Var, bias: Optional[Var], stride=(1, 1), padding=(0, 0), dilation=(1, 1)) -> Var:  # :84-106
    n, c, h, w = x.shape
    o, wc, kh, kw = weight.shape
    assert c == wc
    p = Im2ColParams((kh, kw), tuple(stride), tuple(padding), tuple(dilation))
    oh, ow = p.out_size(h, w)
    assert oh > 0 and ow > 0
    cols = x.im2col(p)
    y = weight.reshape([o, -1]).matmul(cols)
    if bias is not None:
        y = y.add(bias.reshape([o, 1]))
    return y.reshape([n, o, oh, ow])


def _pool2d(x: Var, kernel: int, stride: int, padding: int, is_max: bool) -> Var:  # :121-130
    n, c, h, w = x.shape
    p = Im2ColParams((kernel, kernel), (stride, stride), (padding, padding), (1, 1))
    oh, ow = p.out_size(h, w)
    cols = x.reshape([n * c, 1, h, w]).im2col(p)
    y = cols.max_dims([1], False) if is_max else cols.mean_dims([1], False)
    return y.reshape([n, c, oh, ow])


def max_pool2d(x: Var, kernel: int, stride: int) -> Var:
    return _pool2d(x, kernel, stride, 0, True)


def avg_pool2d(x: Var, kernel: int, stride: int, padding: int) -> Var:
    return _pool2d(x, kernel, stride, padding, False)


def batch_norm(x: Var, running_mean: Optional[Tensor], running_var: Optional[Tensor], weight: Optional[Var],
               bias: Optional[Var], training: bool, momentum: float, eps: float) -> Var:  # :144-180
    c = x.shape[1]
    dims = [d for d in range(x.ndim) if d != 1]
    bshape = [1] * x.ndim
    bshape[1] = c
    if running_mean is not None and running_var is not None and not training:
        mean, var = Var(running_mean.reshape(bshape)), Var(running_var.reshape(bshape))
    else:
        mean = x.mean_dims(dims, True)
        var = x.var_dims(dims, False, True)
        if running_mean is not None and running_var is not None:
            n = x.numel() // c
            unbiased = var.data.mul_scalar(n / (max(n, 2) - 1))
            running_mean.assign(running_mean.mul_scalar(1.0 - momentum).add(mean.data.reshape([c]).mul_scalar(momentum)))
            running_var.assign(running_var.mul_scalar(1.0 - momentum).add(unbiased.reshape([c]).mul_scalar(momentum)))
    y = x.sub(mean).mul(var.add_scalar(eps).sqrt().reciprocal())
    if weight is not None:
        y = y.mul(weight.reshape(bshape))
    if bias is not None:
        y = y.add(bias.reshape(bshape))
    return y


def layer_norm(x: Var, normalized_dims: int, weight: Optional[Var], bias: Optional[Var], eps: float) -> Var:  # :183-195
    dims = list(range(x.ndim - normalized_dims, x.ndim))
    mean = x.mean_dims(dims, True)
    var = x.var_dims(dims, False, True)
    y = x.sub(mean).mul(var.add_scalar(eps).sqrt().reciprocal())
    if weight is not None:
        y = y.mul(weight)
    if bias is not None:
        y = y.add(bias)
    return y


def gelu(x: Var) -> Var:  # :34-36
    return x.mul(x.mul_scalar(math.sqrt(0.5)).erf().add_scalar(1.0)).mul_scalar(0.5)


def gelu_tanh(x: Var) -> Var:  # :39-43
    c = math.sqrt(2.0 / math.pi)
    inner = x.add(x.mul(x).mul(x).mul_scalar(0.044715)).mul_scalar(c)
    return x.mul(inner.tanh().add_scalar(1.0)).mul_scalar(0.5)


def silu(x: Var) -> Var:
    return x.mul(x.sigmoid())


def cross_entropy(logits: Var, target: Tensor) -> Var:  # :200-202
    return logits.cross_entropy(target, "mean", 0.0)


def mse_loss(inp: Var, target: Var) -> Var:  # :224-231
    d = inp.sub(target)
    return d.mul(d).mean()


# -- layers (crates/weta-nn/src/layers.rs) -------------------------------------------------------
def _default_init(weight: Var, bias: Optional[Var]) -> None:
    """layers.rs:19-26: U(-1/sqrt(fan_in), 1/sqrt(fan_in)); the weight's seed is drawn first."""
    fan_in = weight.shape[1] * math.prod(weight.shape[2:])
    bound = 1.0 / math.sqrt(fan_in)
    be = weight.data.backend
    weight.data.assign(Tensor.uniform(weight.shape, -bound, bound, weight.dtype, be))
    if bias is not None:
        bias.data.assign(Tensor.uniform(bias.shape, -bound, bound, bias.dtype, be))


def _param(shape, backend, dtype=DType.F32) -> Var:
    return Var(Tensor.zeros(shape, dtype, backend), requires_grad=True)


class Module:
    training = True

    def parameters(self) -> List[Var]:
        return []

    def named_parameters(self):
        return []

    def buffers(self):
        return []

    def train(self, mode: bool = True):
        self.training = mode
        return self

    def __call__(self, x: Var) -> Var:
        return self.forward(x)


class Linear(Module):
    def __init__(self, in_features: int, out_features: int, backend, dtype=DType.F32):
        self.weight = _param([out_features, in_features], backend, dtype)
        self.bias = _param([out_features], backend, dtype)
        _default_init(self.weight, self.bias)

    def forward(self, x):
        return linear(x, self.weight, self.bias)

    def named_parameters(self):
        return [("weight", self.weight), ("bias", self.bias)]


class Conv2d(Module):
    def __init__(self, cin: int, cout: int, k: int, backend, padding: int = 0, stride: int = 1, dtype=DType.F32):
        self.weight = _param([cout, cin, k, k], backend, dtype)
        self.bias = _param([cout], backend, dtype)
        self.stride, self.padding = stride, padding
        _default_init(self.weight, self.bias)

    def forward(self, x):
        return conv2d(x, self.weight, self.bias, (self.stride,) * 2, (self.padding,) * 2)

    def named_parameters(self):
        return [("weight", self.weight), ("bias", self.bias)]


class BatchNorm2d(Module):
    """layers.rs:235-294"""

    def __init__(self, c: int, backend, dtype=DType.F32, eps: float = 1e-5, momentum: float = 0.1):
        self.weight = Var(Tensor.ones([c], dtype, backend), requires_grad=True)
        self.bias = _param([c], backend, dtype)
        self.running_mean = Tensor.zeros([c], dtype, backend)
        self.running_var = Tensor.ones([c], dtype, backend)
        self.num_batches_tracked = Tensor.zeros([], DType.I64, backend)
        self.eps, self.momentum = eps, momentum

    def forward(self, x):
        if self.training:
            t = self.num_batches_tracked
            t.assign(t.add_scalar(1.0))
        return batch_norm(x, self.running_mean, self.running_var, self.weight, self.bias, self.training,
                          self.momentum, self.eps)

    def named_parameters(self):
        return [("weight", self.weight), ("bias", self.bias)]

    def buffers(self):
        return [("running_mean", self.running_mean), ("running_var", self.running_var),
                ("num_batches_tracked", self.num_batches_tracked)]


class ReLU(Module):
    def forward(self, x):
        return x.relu()


class MaxPool2d(Module):
    def __init__(self, k: int):
        self.k = k

    def forward(self, x):
        return max_pool2d(x, self.k, self.k)


class Flatten(Module):
    def forward(self, x):
        return x.flatten(1, -1)


class Dropout(Module):
    def __init__(self, p: float):
        self.p = p

    def forward(self, x):
        return dropout(x, self.p, self.training)


class Sequential(Module):
    def __init__(self, *layers: Module):
        self.layers = list(layers)

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return x

    def train(self, mode=True):
        for l in self.layers:
            l.train(mode)
        return self

    def named_parameters(self):
        return [(f"{i}.{n}", p) for i, l in enumerate(self.layers) for n, p in l.named_parameters()]

    def parameters(self):
        return [p for _, p in self.named_parameters()]

    def buffers(self):
        return [(f"{i}.{n}", b) for i, l in enumerate(self.layers) for n, b in l.buffers()]

    def state_dict(self):
        d = {n: p.data for n, p in self.named_parameters()}
        d.update(dict(self.buffers()))
        return d


# -- the named models ----------------------------------------------------------------------------
def mlp(backend, dropout_p: float = 0.1, sizes: Sequence[int] = (784, 512, 256, 10)) -> Sequential:
    """784-512-256-10 with ReLU + Dropout after each hidden layer (crates/weta/examples/mnist_mlp.rs:14-33)."""
    layers: List[Module] = [Flatten()]
    for i in range(len(sizes) - 2):
        layers += [Linear(sizes[i], sizes[i + 1], backend), ReLU(), Dropout(dropout_p)]
    layers.append(Linear(sizes[-2], sizes[-1], backend))
    return Sequential(*layers)


def cnn(backend, in_ch: int = 1, hw: int = 28, c1: int = 32, c2: int = 64, hidden: int = 128, classes: int = 10,
        dropout_p: float = 0.25) -> Sequential:
    """crates/weta/examples/mnist_cnn.rs:16-32; the wide variant is c1=128, c2=256, hidden=1024 on 3x32x32."""
    flat = c2 * (hw // 4) * (hw // 4)
    return Sequential(
        Conv2d(in_ch, c1, 3, backend, padding=1), BatchNorm2d(c1, backend), ReLU(), MaxPool2d(2),
        Conv2d(c1, c2, 3, backend, padding=1), BatchNorm2d(c2, backend), ReLU(), MaxPool2d(2),
        Flatten(), Dropout(dropout_p), Linear(flat, hidden, backend), ReLU(), Dropout(dropout_p),
        Linear(hidden, classes, backend))


# -- optimizers (crates/weta-optim/src/lib.rs) ---------------------------------------------------
class SGD:
    """lib.rs:107-125"""

    def __init__(self, params: List[Var], lr: float, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False):
        self.params, self.lr = params, lr
        self.momentum, self.dampening, self.weight_decay, self.nesterov = momentum, dampening, weight_decay, nesterov
        self.buf: List[Optional[Tensor]] = [None] * len(params)

    def zero_grad(self):
        for p in self.params:
            p.grad = None

    def step(self):
        with no_grad():
            for i, p in enumerate(self.params):
                if p.grad is None:
                    continue
                g = p.grad
                if self.weight_decay != 0.0:
                    g = g.add(p.data.mul_scalar(self.weight_decay))
                if self.momentum != 0.0:
                    b = g.copy() if self.buf[i] is None else \
                        self.buf[i].mul_scalar(self.momentum).add(g.mul_scalar(1.0 - self.dampening))
                    g = g.add(b.mul_scalar(self.momentum)) if self.nesterov else b
                    self.buf[i] = b
                p.data.sub_(g.mul_scalar(self.lr))


class Adam:
    """lib.rs:210-239 (`decoupled=True` is AdamW, :276-283)."""

    def __init__(self, params: List[Var], lr: float, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, decoupled=False):
        self.params, self.lr, self.b1, self.b2, self.eps = params, lr, betas[0], betas[1], eps
        self.weight_decay, self.decoupled = weight_decay, decoupled
        self.t = [0] * len(params)
        self.m: List[Optional[Tensor]] = [None] * len(params)
        self.v: List[Optional[Tensor]] = [None] * len(params)

    def zero_grad(self):
        for p in self.params:
            p.grad = None

    def step(self):
        with no_grad():
            for i, p in enumerate(self.params):
                if p.grad is None:
                    continue
                g, theta = p.grad, p.data
                if self.weight_decay != 0.0:
                    if self.decoupled:
                        theta.mul_scalar_(1.0 - self.lr * self.weight_decay)
                    else:
                        g = g.add(theta.mul_scalar(self.weight_decay))
                self.t[i] += 1
                t, b1, b2 = self.t[i], self.b1, self.b2
                m = g.mul_scalar(1.0 - b1) if self.m[i] is None else self.m[i].mul_scalar(b1).add(g.mul_scalar(1.0 - b1))
                gg = g.mul(g).mul_scalar(1.0 - b2)
                v = gg if self.v[i] is None else self.v[i].mul_scalar(b2).add(gg)
                bc1, bc2 = 1.0 - _powi(b1, t), 1.0 - _powi(b2, t)
                denom = v.sqrt().mul_scalar(1.0 / math.sqrt(bc2)).add_scalar(self.eps)
                theta.sub_(m.div(denom).mul_scalar(self.lr / bc1))
                self.m[i], self.v[i] = m, v


def _powi(a: float, n: int) -> float:
    """f64::powi as compiler-rt's __powidf2 evaluates it: square-and-multiply, low bit first."""
    r, b = 1.0, n
    while True:
        if b & 1:
            r *= a
        b //= 2
        if b == 0:
            return r
        a *= a


def AdamW(params, lr, weight_decay=0.01, **kw) -> Adam:
    return Adam(params, lr, weight_decay=weight_decay, decoupled=True, **kw)
