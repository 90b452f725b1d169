"""The fusion planner behind the plain trait (weta_b200/fusion.py + wb_ew_fused): the same stream of trait calls,
issued through `FusingBackend`, must give bit-identical values with fewer launches.  The call streams are the reference's
own (the mirror of weta-tensor / autograd / nn / optim issues them primitive by primitive): element-wise chains with
broadcast operands and shared sub-expressions, in-place assignment, and whole training steps of the two small named
models (crates/weta/examples/mnist_mlp.rs, mnist_cnn.rs)."""
import time

import numpy as np
import pytest

from oracle.mirror import nn
from oracle.mirror.models import build_cnn, mlp_batch, primitive_train_step, synthetic_batch
from oracle.mirror.tensor import Tensor
from weta_b200 import core
from weta_b200.core import DType, manual_seed
from weta_b200.fusion import FusingBackend
from weta_b200.workloads import MNIST_CNN

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(21)


def both(gpu, arr):
    return Tensor.from_numpy(arr, gpu), Tensor.from_numpy(arr, FusingBackend(gpu))


def test_fused_chains_equal_the_separate_launches(gpu):
    fb = FusingBackend(gpu)
    a = RNG.standard_normal((6, 5, 7)).astype(np.float32)
    b = RNG.standard_normal((6, 5, 7)).astype(np.float32)
    row = RNG.standard_normal((7,)).astype(np.float32)
    col = RNG.standard_normal((6, 1, 1)).astype(np.float32)
    out = {}
    for name, be in (("plain", gpu), ("fused", fb)):
        A, B, R, C = (Tensor.from_numpy(x, be) for x in (a, b, row, col))
        shared = A.mul(B).add_scalar(0.5)                       # used twice below
        y1 = shared.relu().sub(R.broadcast_to([6, 5, 7])).mul(C.broadcast_to([6, 5, 7])).tanh()
        y2 = shared.mul(shared).sqrt().add(A.transpose(0, 2).contiguous().transpose(0, 2))  # a strided operand
        y3 = y1.gt_scalar(0.1).mul_scalar(1.0 / 0.9).mul(y2)     # dropout-like tail on top of both
        z = A.transpose(1, 2).exp().mul(B.transpose(1, 2))        # the whole chain runs over a transposed index space
        long = A
        for i in range(60):                                       # longer than one program: must be split
            long = long.mul_scalar(1.0 + 1e-3 * i).add(B)
        out[name] = [t.numpy() for t in (y1, y2, y3, z, long, shared)]
    for i, (p, f) in enumerate(zip(out["plain"], out["fused"])):
        assert p.shape == f.shape and np.array_equal(p, f, equal_nan=True), i
    assert fb.programs < fb.ops_deferred / 3, (fb.programs, fb.ops_deferred)


def test_in_place_assignment_sees_and_hides_the_right_values(gpu):
    """`theta.sub_(step)` writes the pending expression straight over theta; an expression that read theta earlier must
    have been evaluated first, and a handle that aliases theta must keep its value when theta changes again."""
    fb = FusingBackend(gpu)
    t0 = RNG.standard_normal(1000).astype(np.float32)
    g = RNG.standard_normal(1000).astype(np.float32)
    res = {}
    for name, be in (("plain", gpu), ("fused", fb)):
        theta, grad = Tensor.from_numpy(t0.copy(), be), Tensor.from_numpy(g, be)
        before = theta.mul_scalar(2.0)          # pending, reads theta
        theta.sub_(grad.mul_scalar(0.1))        # in place
        mid = theta.add_scalar(0.0).mul_scalar(1.0)
        kept = theta.sub(grad.mul_scalar(0.5))  # pending
        theta.assign(kept)                      # written straight into theta; `kept` now shares its storage
        theta.sub_(grad)                        # theta changes again: `kept` must not
        res[name] = [x.numpy() for x in (before, mid, kept, theta)]
    for p, f in zip(res["plain"], res["fused"]):
        assert np.array_equal(p, f)


def _mlp_steps(be, steps):
    manual_seed(42)
    model = nn.mlp(be, 0.1)
    opt = nn.Adam(model.parameters(), 1e-3)
    core._global_rng = core.Pcg(4242)
    losses = [primitive_train_step(model, opt, *mlp_batch(128, s, be)) for s in range(steps)]
    return losses, [p.numpy() for p in model.parameters()]


def _cnn_steps(be, steps):
    model = build_cnn(MNIST_CNN, be, 42)
    opt = nn.Adam(model.parameters(), 1e-3)
    core._global_rng = core.Pcg(777)
    losses = [primitive_train_step(model, opt, *synthetic_batch(MNIST_CNN, 64, s, 0, be)) for s in range(steps)]
    return losses, [p.numpy() for p in model.parameters()] + [b.numpy() for _, b in model.buffers()]


@pytest.mark.parametrize("which", ["mlp 784-512-256-10 batch 128", "cnn-mnist-422k batch 64"])
def test_unmodified_training_step_through_the_planner(gpu, report, which):
    """Three Adam steps of a named model in primitive mode, once through the plain backend and once through the planner:
    identical losses and state, launches per step counted on the backend."""
    run = _mlp_steps if which.startswith("mlp") else _cnn_steps
    stats = {}
    results = {}
    for name in ("plain", "fused"):
        be = gpu if name == "plain" else FusingBackend(gpu)
        run(be, 1)  # warm the arena
        gpu.synchronize()
        l0, t0 = gpu.launch_count(), time.perf_counter()
        results[name] = run(be, 3)
        gpu.synchronize()
        stats[name] = {"launches_per_step": (gpu.launch_count() - l0) / 3.0, "ms_per_step": (time.perf_counter() - t0) / 3.0 * 1e3}
        if name == "fused":
            stats[name].update(trait_calls_deferred=be.ops_deferred, fused_launches=be.programs, calls_in_fused_launches=be.ops_fused)
    report(f"primitive-mode step through the fusion planner: {which}", **stats)
    assert results["plain"][0] == results["fused"][0]
    for p, f in zip(results["plain"][1], results["fused"][1]):
        assert np.array_equal(p, f)
    assert stats["fused"]["launches_per_step"] < 0.6 * stats["plain"]["launches_per_step"], stats
