"""TEST INFRASTRUCTURE, NOT PRODUCT CODE: the named models in primitive mode and their synthetic inputs as tensors.

Synthetic data stands in for MNIST / CIFAR-10 (neither is available offline): tensors of the same
shape and value range, drawn from the counter RNG so every backend sees identical inputs
without any file moving.
"""
from __future__ import annotations

from typing import Tuple

from weta_b200.core import Distribution, DType, manual_seed
from weta_b200.workloads import CnnConfig, batch_seeds

from . import nn
from .autograd import Var
from .tensor import Tensor


def synthetic_batch(cfg: CnnConfig, batch: int, step: int, rank: int, backend) -> Tuple[Tensor, Tensor]:
    """Images U[0,1) and uniform labels, seeded by (step, rank): the tensors `weta_b200.workloads.synthetic_batch_device`
    draws on the GPU, here on any backend object."""
    sx, sy = batch_seeds(step, rank)
    x = Tensor.random_seeded([batch, cfg.in_ch, cfg.hw, cfg.hw], Distribution.uniform(0.0, 1.0), DType.F32, backend, sx)
    y = Tensor.random_seeded([batch], Distribution.uniform(0.0, float(cfg.classes)), DType.I64, backend, sy)
    return x, y


def build_cnn(cfg: CnnConfig, backend, seed: int = 42) -> nn.Sequential:
    manual_seed(seed)
    return nn.cnn(backend, cfg.in_ch, cfg.hw, cfg.c1, cfg.c2, cfg.hidden, cfg.classes, cfg.dropout)


def primitive_train_step(model: nn.Sequential, opt, x: Tensor, y: Tensor, grad_hook=None) -> float:
    """One step exactly as crates/weta/examples/mnist_cnn.rs:63-73 runs it: forward, cross-entropy,
    zero_grad, backward, step, loss.item().  `grad_hook(params)` runs between backward and the
    optimizer (the data-parallel gradient average)."""
    loss = nn.cross_entropy(model(Var(x)), y)
    opt.zero_grad()
    loss.backward()
    if grad_hook is not None:
        grad_hook(model.parameters())
    opt.step()
    return loss.item()


def mlp_batch(batch: int, step: int, backend) -> Tuple[Tensor, Tensor]:
    """Config-1 inputs: pixels k/255 with k uniform in 0..255, labels uniform in 0..9."""
    px = Tensor.random_seeded([batch, 784], Distribution.uniform(0.0, 256.0), DType.I64, backend, 10_000 + step)
    x = px.to_dtype(DType.F32).mul_scalar(1.0 / 255.0)
    y = Tensor.random_seeded([batch], Distribution.uniform(0.0, 10.0), DType.I64, backend, 20_000 + step)
    return x, y
