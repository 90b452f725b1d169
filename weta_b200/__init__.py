"""weta_b200: a B200-native implementation of weta's tensor-operator backend.

`weta_b200.backend.B200Backend` binds the C ABI in include/weta_b200.h (hand-written sm_100a
kernels) with the method set of `weta_core::Backend`; `trainer` drives the fused training step
and its data-parallel form; `core` holds the vocabulary (dtypes, op codes, layouts, host RNG).
"""
from .core import (BinaryOp, Distribution, DType, Im2ColParams, Layout, Pcg, ReduceOp, UnaryOp, manual_seed)  # noqa: F401
