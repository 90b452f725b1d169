"""The benchmark workloads: synthetic inputs and the primitive-mode training step.

Synthetic data stands in for MNIST / CIFAR-10 (neither is available offline): tensors of the same
shape and value range, drawn from the counter RNG so every backend sees identical inputs
without any file moving.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

from . import nn
from .autograd import Var
from .core import Distribution, DType, manual_seed
from .tensor import Tensor


@dataclass(frozen=True)
class CnnConfig:
    name: str
    in_ch: int
    hw: int
    c1: int
    c2: int
    hidden: int
    classes: int = 10
    dropout: float = 0.25

    def num_params(self) -> int:
        flat = self.c2 * (self.hw // 4) ** 2
        return (self.c1 * self.in_ch * 9 + self.c1 + 2 * self.c1 + self.c2 * self.c1 * 9 + self.c2 + 2 * self.c2 +
                self.hidden * flat + self.hidden + self.classes * self.hidden + self.classes)

    def train_flops_per_sample(self) -> float:
        """2*M*N*K of every contraction, forward + both gradients (conv1 has no input gradient)."""
        hw = self.hw * self.hw
        conv1 = 2 * self.c1 * self.in_ch * 9 * hw
        conv2 = 2 * self.c2 * self.c1 * 9 * (hw // 4)
        fc1 = 2 * self.hidden * self.c2 * (hw // 16)
        fc2 = 2 * self.classes * self.hidden
        return 2 * conv1 + 3 * (conv2 + fc1 + fc2)


# crates/weta/examples/mnist_cnn.rs:16-32 (422k parameters) and the widened data-parallel variant.
MNIST_CNN = CnnConfig("cnn-mnist-422k", 1, 28, 32, 64, 128)
WIDE_CNN = CnnConfig("cnn-wide-17M", 3, 32, 128, 256, 1024)


def synthetic_batch(cfg: CnnConfig, batch: int, step: int, rank: int, backend) -> Tuple[Tensor, Tensor]:
    """Images U[0,1) and uniform labels, seeded by (step, rank)."""
    seed = 10_000 + 1_000_003 * rank + step
    x = Tensor.random_seeded([batch, cfg.in_ch, cfg.hw, cfg.hw], Distribution.uniform(0.0, 1.0), DType.F32, backend, seed)
    y = Tensor.random_seeded([batch], Distribution.uniform(0.0, float(cfg.classes)), DType.I64, backend, seed + 500_000_000)
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
