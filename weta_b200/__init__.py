"""weta_b200: a B200-native implementation of weta's tensor-operator backend.

`weta_b200.backend.B200Backend` binds the C ABI in include/weta_b200.h (hand-written sm_100a
kernels); `tensor`, `autograd` and `nn` mirror the call sites of the reference above that
boundary; `trainer` drives the fused training step and its data-parallel wrapper.
"""
from .core import (BinaryOp, Distribution, DType, Im2ColParams, Layout, Pcg, ReduceOp, UnaryOp, manual_seed)  # noqa: F401
from .tensor import Tensor, allclose  # noqa: F401
