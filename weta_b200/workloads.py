"""The benchmark workloads: model configurations and synthetic inputs drawn on the device.

Synthetic data stands in for MNIST / CIFAR-10 (neither is available offline): tensors of the same
shape and value range, drawn from the counter RNG (`Backend::random`, crates/weta-core/src/backend.rs:97-105)
so every backend sees identical inputs without any file moving.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

from .core import Distribution, DType, Layout


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


def batch_seeds(step: int, rank: int) -> Tuple[int, int]:
    """Counter-RNG seeds of the images and the labels of one synthetic batch."""
    seed = 10_000 + 1_000_003 * rank + step
    return seed, seed + 500_000_000


def synthetic_batch_device(cfg: CnnConfig, batch: int, step: int, rank: int, backend):
    """Images U[0,1) f32 [batch, in_ch, hw, hw] and uniform i64 labels [batch] as device storages, seeded by
    (step, rank).  Integer tensors are drawn as f64 and cast (crates/weta-tensor/src/random.rs:104-110)."""
    sx, sy = batch_seeds(step, rank)
    x = backend.random(batch * cfg.in_ch * cfg.hw * cfg.hw, DType.F32, Distribution.uniform(0.0, 1.0), sx)
    yf = backend.random(batch, DType.F64, Distribution.uniform(0.0, float(cfg.classes)), sy)
    y = backend.cast(yf, Layout.contiguous([batch]), DType.F64, DType.I64)
    return x, y
