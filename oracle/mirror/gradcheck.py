"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: f64 central-difference gradient check, as crates/weta-autograd/src/gradcheck.rs:46-90.

The loss is sum(f(inputs) * r) for a fixed random r; every element of every input is nudged by +-eps through a
one-element in-place fill (a strided `copy_strided` on the backend), and the analytic gradient must agree with
(loss+ - loss-) / (2 eps) to `tol` relative to max(1, |analytic|, |numeric|)."""
from __future__ import annotations

from typing import Callable, List, Optional

from weta_b200.core import DType

from .autograd import Var, no_grad
from .tensor import Tensor


def _element(t: Tensor, flat: int) -> Tensor:
    """A one-element view of element `flat` (row-major) of t (gradcheck.rs:34-42)."""
    v = t
    for d in reversed(range(t.ndim)):
        n = t.shape[d]
        v = v.narrow(d, flat % n, 1)
        flat //= n
    return v


def gradcheck(f: Callable[[List[Var]], Var], inputs: List[Var], eps: float = 1e-5, tol: float = 1e-6) -> Optional[str]:
    """None when every gradient checks out, else a description of the first mismatch."""
    for i, x in enumerate(inputs):
        if x.dtype != DType.F64:
            return f"gradcheck: input {i} is not f64"
    y = f(inputs)
    r = Var(Tensor.randn(list(y.shape), DType.F64, y.data.backend))
    loss = lambda xs: f(xs).mul(r).sum()
    for x in inputs:
        x.grad = None
    loss(inputs).backward()
    for i, x in enumerate(inputs):
        if not x.requires_grad:
            continue
        analytic = x.grad.numpy().reshape(-1) if x.grad is not None else [0.0] * x.numel()
        with no_grad():
            for k, a in enumerate(analytic):
                e = _element(x.data, k)
                orig = e.item()
                e.fill_(orig + eps)
                plus = loss(inputs).item()
                e.fill_(orig - eps)
                minus = loss(inputs).item()
                e.fill_(orig)
                numeric = (plus - minus) / (2.0 * eps)
                err = abs(a - numeric) / max(1.0, abs(a), abs(numeric))
                if not err <= tol:  # written so a NaN error fails too
                    return (f"gradcheck: input {i} (shape {x.shape}), element {k}: analytic {a:.10e}, numeric {numeric:.10e}, "
                            f"relative error {err:.3e}")
    return None
