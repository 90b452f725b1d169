"""Fused extension ops and the fused training step against the CPU oracle running the reference's
primitive sequences (the op-by-op definitions in crates/weta-nn/src/functional.rs,
crates/weta-autograd/src/ops.rs and crates/weta-optim/src/lib.rs)."""
import ctypes

import numpy as np
import pytest

from weta_b200 import core
from oracle.mirror import nn
from oracle.mirror.autograd import Var
from weta_b200.core import Distribution, DType, manual_seed
from oracle.mirror.tensor import Tensor, allclose
from weta_b200.trainer import FusedTrainer, _declare, cnn_specs, mlp_specs
from weta_b200.workloads import MNIST_CNN, CnnConfig
from oracle.mirror.models import build_cnn, mlp_batch, primitive_train_step, synthetic_batch

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(7)
FP32, TF32, TF32X3 = 2, 1, 0


def dev(gpu, arr):
    t = Tensor.from_numpy(np.ascontiguousarray(arr), gpu)
    return t, t.storage.ptr


def empty(gpu, n, dt=DType.F32):
    s = gpu.alloc(int(n), dt)
    return s, s.ptr


def fetch(gpu, storage, shape, dt=DType.F32):
    from weta_b200.core import Layout
    return gpu.to_host(storage, Layout.contiguous(shape), dt).reshape(shape)


def test_dropout_is_bit_identical_to_the_primitive_chain(oracle, gpu):
    _declare(gpu.lib)
    n, p, seed = (1 << 20) + 3, 0.1, 42
    x = RNG.standard_normal(n).astype(np.float32)
    xo = Tensor.from_numpy(x, oracle)
    mask_o = Tensor.random_seeded([n], Distribution.uniform(0.0, 1.0), DType.F32, oracle, seed).gt_scalar(p).mul_scalar(1.0 / (1.0 - p))
    want = xo.mul(mask_o).numpy()
    (xt, xp), (ys, yp), (ms, mp) = dev(gpu, x), empty(gpu, n), empty(gpu, n)
    gpu.check(gpu.lib.wb_dropout_fwd(gpu.handle, xp, yp, n, p, seed))
    gpu.check(gpu.lib.wb_dropout_mask(gpu.handle, mp, n, p, seed))
    assert np.array_equal(fetch(gpu, ys, (n,)), want)
    mask = fetch(gpu, ms, (n,))
    assert np.array_equal(mask, mask_o.numpy())
    assert set(np.unique(mask).tolist()) == {0.0, float(np.float32(1.0 / 0.9))}
    # the same mask through the trait ops on the GPU
    mask_g = Tensor.random_seeded([n], Distribution.uniform(0.0, 1.0), DType.F32, gpu, seed).gt_scalar(p).mul_scalar(1.0 / (1.0 - p))
    assert np.array_equal(mask_g.numpy(), mask)


def test_dropout_mask_2_pow_28_seed_42(oracle, gpu):
    """The full-size mask fill: 2^28 elements, p = 0.1, seed 42, compared element for element."""
    _declare(gpu.lib)
    n, p = 1 << 28, 0.1
    ms, mp = empty(gpu, n)
    gpu.check(gpu.lib.wb_dropout_mask(gpu.handle, mp, n, p, 42))
    got = fetch(gpu, ms, (n,))
    want = Tensor.random_seeded([n], Distribution.uniform(0.0, 1.0), DType.F32, oracle, 42).gt_scalar(p).mul_scalar(1.0 / (1.0 - p)).numpy()
    assert int((got != want).sum()) == 0


def test_softmax_cross_entropy(oracle, gpu):
    _declare(gpu.lib)
    for rows, cols in [(128, 10), (257, 1000), (64, 33)]:
        z = (RNG.standard_normal((rows, cols)) * 3).astype(np.float32)
        y = RNG.integers(0, cols, rows).astype(np.int64)
        zv = Var(Tensor.from_numpy(z, oracle), requires_grad=True)
        loss = zv.cross_entropy(Tensor.from_numpy(y, oracle))
        loss.backward()
        (zt, zp), (yt, yp) = dev(gpu, z), dev(gpu, y)
        (ps, pp), (ds, dp), (ls, lp) = empty(gpu, rows * cols), empty(gpu, rows * cols), empty(gpu, 1)
        gpu.check(gpu.lib.wb_softmax_ce(gpu.handle, zp, yp, rows, cols, pp, dp, None, lp, 1.0))
        assert abs(fetch(gpu, ls, (1,))[0] - loss.item()) <= 1e-5 * max(1.0, abs(loss.item()))
        assert allclose(fetch(gpu, ds, (rows, cols)), zv.grad.numpy(), 1e-4, 1e-7)
        assert allclose(fetch(gpu, ps, (rows, cols)), Tensor.from_numpy(z, oracle).softmax(1).numpy(), 1e-4, 1e-7)


def _oracle_bn(oracle, x, gamma, beta, upstream=None, pool=False):
    xv = Var(Tensor.from_numpy(x, oracle), requires_grad=True)
    gv = Var(Tensor.from_numpy(gamma, oracle), requires_grad=True)
    bv = Var(Tensor.from_numpy(beta, oracle), requires_grad=True)
    c = x.shape[1]
    rm, rv = Tensor.zeros([c], DType.F32, oracle), Tensor.ones([c], DType.F32, oracle)
    y = nn.batch_norm(xv, rm, rv, gv, bv, True, 0.1, 1e-5)
    if pool:
        y = nn.max_pool2d(y.relu(), 2, 2)
    if upstream is not None:
        y.mul(Var(Tensor.from_numpy(upstream, oracle))).sum().backward()
    return y.numpy(), rm.numpy(), rv.numpy(), xv.grad, gv.grad, bv.grad


def test_batch_norm_2d(oracle, gpu):
    _declare(gpu.lib)
    n, c, h, w = 6, 5, 7, 9
    x = (RNG.standard_normal((n, c, h, w)) * 2 + 3).astype(np.float32)
    gamma, beta = RNG.standard_normal(c).astype(np.float32), RNG.standard_normal(c).astype(np.float32)
    up = RNG.standard_normal((n, c, h, w)).astype(np.float32)
    y_o, rm_o, rv_o, dx_o, dg_o, db_o = _oracle_bn(oracle, x, gamma, beta, up)
    (xt, xp), (gt, gp), (bt, bp), (ut, upp) = dev(gpu, x), dev(gpu, gamma), dev(gpu, beta), dev(gpu, up)
    (rmt, rmp), (rvt, rvp) = dev(gpu, np.zeros(c, np.float32)), dev(gpu, np.ones(c, np.float32))
    (ys, yp), (ms, mp), (rs, rp) = empty(gpu, x.size), empty(gpu, c), empty(gpu, c)
    gpu.check(gpu.lib.wb_bn2d_fwd(gpu.handle, xp, n, c, h * w, gp, bp, rmp, rvp, 0.1, 1e-5, yp, mp, rp))
    assert allclose(fetch(gpu, ys, x.shape), y_o, 1e-5, 1e-5)
    assert allclose(rmt.numpy(), rm_o, 1e-6, 1e-6) and allclose(rvt.numpy(), rv_o, 1e-5, 1e-6)
    (dxs, dxp), (dgs, dgp), (dbs, dbp) = empty(gpu, x.size), empty(gpu, c), empty(gpu, c)
    gpu.check(gpu.lib.wb_bn2d_bwd(gpu.handle, xp, upp, n, c, h * w, gp, mp, rp, dxp, dgp, dbp))
    assert allclose(fetch(gpu, dxs, x.shape), dx_o.numpy(), 1e-4, 2e-5)
    assert allclose(fetch(gpu, dgs, (c,)), dg_o.numpy(), 1e-4, 1e-4)
    assert allclose(fetch(gpu, dbs, (c,)), db_o.numpy(), 1e-4, 1e-4)


@pytest.mark.parametrize("shape", [(5, 4, 8, 12), (3, 6, 4, 16), (2, 3, 6, 8), (2, 3, 4, 6)])
def test_bn_relu_pool_block_with_ties(oracle, gpu, shape):
    """Widths 16 and 8 take the four-pooled-values-per-thread forward kernel (72 and 18 items: part-filled warps),
    12 and 16 and 8 the paired backward kernels, 6 the scalar ones."""
    _declare(gpu.lib)
    n, c, h, w = shape
    x = RNG.standard_normal((n, c, h, w)).astype(np.float32)
    x[0, 0, 0:2, 0:2] = 1.5          # a window of four equal positives: the gradient splits four ways
    x[1, 2, 2:4, 4:6] = [[0.7, 0.7], [-1.0, 0.1]]  # two-way tie
    gamma = (np.abs(RNG.standard_normal(c)) + 0.5).astype(np.float32)
    beta = (RNG.standard_normal(c) * 0.1).astype(np.float32)
    up = RNG.standard_normal((n, c, h // 2, w // 2)).astype(np.float32)
    y_o, rm_o, rv_o, dx_o, dg_o, db_o = _oracle_bn(oracle, x, gamma, beta, up, pool=True)
    (xt, xp), (gt, gp), (bt, bp), (ut, upp) = dev(gpu, x), dev(gpu, gamma), dev(gpu, beta), dev(gpu, up)
    (rmt, rmp), (rvt, rvp) = dev(gpu, np.zeros(c, np.float32)), dev(gpu, np.ones(c, np.float32))
    (ys, yp), (ms, mp), (rs, rp) = empty(gpu, up.size), empty(gpu, c), empty(gpu, c)
    gpu.check(gpu.lib.wb_bn_relu_pool_fwd(gpu.handle, xp, n, c, h, w, gp, bp, rmp, rvp, 0.1, 1e-5, yp, mp, rp))
    assert allclose(fetch(gpu, ys, up.shape), y_o, 1e-5, 1e-5)
    assert allclose(rvt.numpy(), rv_o, 1e-5, 1e-6)
    (dxs, dxp), (dgs, dgp), (dbs, dbp), (dcs, dcp) = empty(gpu, x.size), empty(gpu, c), empty(gpu, c), empty(gpu, c)
    gpu.check(gpu.lib.wb_bn_relu_pool_bwd(gpu.handle, xp, upp, n, c, h, w, gp, bp, mp, rp, dxp, dgp, dbp, dcp))
    dx = fetch(gpu, dxs, x.shape)
    assert allclose(dx, dx_o.numpy(), 1e-4, 2e-5)
    assert allclose(fetch(gpu, dgs, (c,)), dg_o.numpy(), 1e-4, 1e-4)
    assert allclose(fetch(gpu, dbs, (c,)), db_o.numpy(), 1e-4, 1e-4)
    assert allclose(fetch(gpu, dcs, (c,)), dx.sum(axis=(0, 2, 3)), 1e-3, 1e-4)


@pytest.mark.parametrize("wd,decoupled", [(0.0, False), (0.1, False), (0.1, True)])
def test_adam_is_bit_identical_to_the_primitive_chain(oracle, gpu, wd, decoupled):
    _declare(gpu.lib)
    n = 10007
    p0 = RNG.standard_normal(n).astype(np.float32)
    grads = [RNG.standard_normal(n).astype(np.float32) * s for s in (1.0, 1e-3, 10.0)]
    pv = Var(Tensor.from_numpy(p0.copy(), oracle), requires_grad=True)
    opt = nn.Adam([pv], 1e-3, weight_decay=wd, decoupled=decoupled)
    (tt, tp) = dev(gpu, p0)
    (mt, mp), (vt, vp) = dev(gpu, np.zeros(n, np.float32)), dev(gpu, np.zeros(n, np.float32))
    for step, g in enumerate(grads, 1):
        pv.grad = Tensor.from_numpy(g, oracle)
        opt.step()
        gt, gp = dev(gpu, g)
        gpu.check(gpu.lib.wb_adam_step(gpu.handle, tp, gp, mp, vp, n, step, 1e-3, 0.9, 0.999, 1e-8, wd, int(decoupled), 1.0))
        assert np.array_equal(tt.numpy(), pv.numpy()), f"step {step}"
        assert np.array_equal(mt.numpy(), opt.m[0].numpy()) and np.array_equal(vt.numpy(), opt.v[0].numpy())


def _adam_params_close(name, got, want, steps, lr, frac_allowed=2e-3):
    d = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert d.max() <= 2 * steps * lr * 1.01, f"{name}: max |diff| {d.max()}"
    frac = float((d > 1e-5 + 1e-4 * np.abs(want)).mean())
    assert frac < frac_allowed, f"{name}: {frac:.2%} of elements differ by more than 1e-5"


@pytest.mark.parametrize("mode", [FP32, TF32X3])
def test_fused_mlp_matches_the_primitive_step(oracle, gpu, mode):
    """784-512-256-10, ReLU + Dropout(0.1), batch 128, Adam 1e-3, seed 42, 10 steps."""
    manual_seed(42)
    ref = nn.mlp(oracle, 0.1)
    opt = nn.Adam(ref.parameters(), 1e-3)
    manual_seed(42)
    tr = FusedTrainer(gpu, mlp_specs(), 128, (784, 1, 1), lr=1e-3, matmul_mode=mode)
    tr.init_from_global_rng()
    for i, p in enumerate(ref.parameters()):
        assert np.array_equal(tr.get_param(i), p.numpy().reshape(-1)), f"initial parameter {i}"
    state_after_init = (core.global_rng().state,)
    losses = []
    for be_name in ("oracle", "fused"):
        core.global_rng().state = state_after_init[0]
        for step in range(10):
            x, y = mlp_batch(128, step, oracle)
            if be_name == "oracle":
                l = primitive_train_step(ref, opt, x, y)
                if step == 0:
                    g0 = [p.grad.numpy().reshape(-1) for p in ref.parameters()]
            else:
                tr.stage(x.numpy(), y.numpy())
                tr.forward_backward()
                if step == 0:
                    for i, g in enumerate(g0):
                        got = tr.get_grad(i)
                        assert np.abs(got - g).max() <= 2e-4 * max(np.abs(g).max(), 1e-6), f"grad {i}"
                tr.adam_step()
                l = tr.loss()
            losses.append(l)
    for a, b in zip(losses[:10], losses[10:]):
        assert abs(a - b) < 2e-4, (losses[:10], losses[10:])
    for i, (n, p) in enumerate(ref.named_parameters()):
        # 3xTF32 gradients carry ~1e-5 relative error; where |g| is itself tiny Adam's sign-like step
        # turns that into a different step, so more elements drift than in FP32 mode (the hard bound holds).
        _adam_params_close(n, tr.get_param(i), p.numpy().reshape(-1), 10, 1e-3, 5e-3 if mode == FP32 else 0.15)
    gpu.gemm_check()
    tr.close()


@pytest.mark.parametrize("mode", [FP32, TF32X3])
def test_fused_cnn_matches_the_primitive_step(oracle, gpu, mode):
    """The 422k-parameter CNN (conv-BN-ReLU-pool x2, dropout, fc 128, dropout, fc 10), batch 64, 3 Adam steps."""
    _check_cnn(oracle, gpu, MNIST_CNN, 64, mode)


def test_fused_cnn_tf32_matches_the_oracle_on_tf32_operands(tf32_oracle, gpu, report):
    """The same model with one-product TF32 contractions, against the oracle reading its matmul operands as TF32."""
    _check_cnn(tf32_oracle, gpu, MNIST_CNN, 64, TF32, tf32_operands=True, report=report, name="cnn-mnist-422k batch 64")


def test_fused_cnn_with_implicit_gemm_convolution(tf32_oracle, gpu, report):
    """A CNN whose second block (128 -> 32 channels on 8x8) takes the implicit-GEMM convolution for forward,
    weight gradient and input gradient; the first block (3 channels) keeps im2col.  The oracle's contractions read
    their operands as TF32, so the two sides differ by accumulation error only and the bounds are tight."""
    cfg = CnnConfig("cnn-implicit", 3, 16, 128, 32, 64)
    _check_cnn(tf32_oracle, gpu, cfg, 16, TF32, tf32_operands=True, report=report, name="cnn-implicit batch 16")


def test_implicit_and_explicit_convolution_paths_agree(gpu, monkeypatch):
    """Same TF32 operand rounding, different accumulation order: the two paths' gradients agree to 1e-3 in
    the 2-norm over one forward/backward of the same batch (measured 2e-4 on the first block's weight)."""
    cfg = CnnConfig("cnn-implicit", 3, 16, 128, 32, 64)
    grads = []
    for explicit in ("1", "0"):
        monkeypatch.setenv("WETA_B200_EXPLICIT_CONV", explicit)
        manual_seed(42)
        tr = FusedTrainer(gpu, cnn_specs(cfg), 32, (cfg.in_ch, cfg.hw, cfg.hw), lr=1e-3, matmul_mode=TF32)
        tr.init_from_global_rng()
        x, y = synthetic_batch(cfg, 32, 0, 0, gpu)
        tr.stage(x.numpy(), y.numpy())
        tr.forward_backward()
        grads.append(([tr.get_grad(i) for i in range(12)], tr.loss()))
        tr.close()
    (ge, le), (gi, li) = grads
    assert abs(le - li) < 1e-5
    for i, (a, b) in enumerate(zip(ge, gi)):
        if i in (1, 5):
            continue  # conv biases before BatchNorm: rounding noise around a zero gradient
        assert np.linalg.norm(a - b) <= 1e-3 * np.linalg.norm(a), i


def _check_cnn(oracle, gpu, cfg, batch, mode, grad_norm_tol=5e-2, loss_tol=None, tf32_operands=False, steps=3, report=None, name=""):
    """Fused trainer against the oracle's primitive step.  With tf32_operands the oracle passed in truncates its matmul
    operands to TF32 (fixture tf32_oracle), so both sides contract the same operand values and each contraction agrees
    to ~1e-6.  What is left end to end is the network's own conditioning: activations that differ in the last f32
    place land in different TF32 steps for one element in a few thousand, and the gradients of a conv-BN stack at a
    small batch amplify any perturbation (BatchNorm makes the loss invariant to each channel's weight scale, so those
    gradients are differences of much larger terms; in FP32 mode the first convolution's weight gradient already
    differs from the oracle's by 1e-3 with every contraction exact to 1e-7).  Bounds: 5e-5 on the first loss and
    grad_norm_tol (default 3e-3) on every gradient's 2-norm, against 3e-3 and 5e-2..2e-1 for a plain-f32 oracle."""
    ref = build_cnn(cfg, oracle, 42)
    opt = nn.Adam(ref.parameters(), 1e-3)
    manual_seed(42)
    tr = FusedTrainer(gpu, cnn_specs(cfg), batch, (cfg.in_ch, cfg.hw, cfg.hw), lr=1e-3, matmul_mode=mode)
    tr.init_from_global_rng()
    names = [n for n, _ in ref.named_parameters()]
    for i, p in enumerate(ref.parameters()):
        assert np.array_equal(tr.get_param(i), p.numpy().reshape(-1)), f"initial {names[i]}"
    rng_state = core.global_rng().state
    tol_loss, tol_grad = {FP32: (2e-4, 2e-3), TF32X3: (2e-4, 2e-3), TF32: (3e-3, 3e-2)}[mode]
    if tf32_operands:
        tol_loss = 2e-4 if batch < 32 else 5e-5
        grad_norm_tol = 3e-3 if grad_norm_tol == 5e-2 else grad_norm_tol
        loss_tol = 2e-3 if loss_tol is None else loss_tol
    ref_losses, ref_g0 = [], None
    for step in range(steps):
        x, y = synthetic_batch(cfg, batch, step, 0, oracle)
        ref_losses.append(primitive_train_step(ref, opt, x, y))
        if step == 0:
            ref_g0 = [p.grad.numpy().reshape(-1) for p in ref.parameters()]
    core.global_rng().state = rng_state
    seen = {"loss": [], "grad_norm_err": {}}
    for step in range(steps):
        x, y = synthetic_batch(cfg, batch, step, 0, oracle)
        tr.stage(x.numpy(), y.numpy())
        tr.forward_backward()
        if step == 0:
            for i, g in enumerate(ref_g0):
                if names[i] in ("0.bias", "4.bias"):
                    continue  # conv bias before BatchNorm: the true gradient is zero, both sides hold rounding noise
                got = tr.get_grad(i)
                if mode == TF32:
                    # One-product TF32 against a plain-f32 oracle perturbs activations by ~1e-3, enough to flip a few
                    # max-pool winners and ReLU gates; single entries then move a lot, so compare in the 2-norm.
                    err = float(np.linalg.norm(got - g) / np.linalg.norm(g))
                    seen["grad_norm_err"][names[i]] = err
                    assert err <= grad_norm_tol, f"grad {names[i]}: relative 2-norm error {err}"
                else:
                    assert np.abs(got - g).max() <= tol_grad * max(np.abs(g).max(), 1e-6), f"grad {names[i]}"
        tr.adam_step()
        # later steps: after an Adam step the sign-like update amplifies gradient noise where |g| is tiny
        seen["loss"].append((tr.loss(), ref_losses[step]))
        bound = tol_loss if step == 0 or loss_tol is None else loss_tol * max(1.0, abs(ref_losses[step]))
        assert abs(tr.loss() - ref_losses[step]) < bound, (step, tr.loss(), ref_losses)
    if report is not None:
        report(f"fused CNN vs oracle: {name}", mode=mode, tf32_operands=tf32_operands, losses=seen["loss"], grad_norm_err=seen["grad_norm_err"])
    if mode != TF32:
        for i, (n, p) in enumerate(ref.named_parameters()):
            if n in ("0.bias", "4.bias"):
                assert np.abs(tr.get_param(i) - p.numpy().reshape(-1)).max() <= 2 * 3 * 1e-3 * 1.01
            else:
                _adam_params_close(n, tr.get_param(i), p.numpy().reshape(-1), 3, 1e-3, 2e-2)
        bufs = dict(ref.buffers())
        for k, idx in ((0, "1"), (1, "5")):
            rm, rv = tr.bn_buffers(k)
            assert allclose(rm, bufs[f"{idx}.running_mean"].numpy(), 0.0, 3e-3)
            assert allclose(rv, bufs[f"{idx}.running_var"].numpy(), 1e-3, 1e-5)
    gpu.gemm_check()
    tr.close()


def test_bucket_callback_covers_the_arena(gpu):
    cfg = CnnConfig("tiny", 3, 8, 8, 16, 32)
    manual_seed(1)
    tr = FusedTrainer(gpu, cnn_specs(cfg), 16, (3, 8, 8), matmul_mode=FP32)
    tr.init_from_global_rng()
    seen = []
    base = tr.grads_ptr()
    tr.set_bucket_callback(lambda ptr, n: seen.append(((ptr - base) // 4, n)))
    x = RNG.random((16, 3, 8, 8)).astype(np.float32)
    y = RNG.integers(0, 10, 16)
    tr.stage(x, y)
    tr.forward_backward()
    gpu.synchronize()
    assert seen[0][0] == 0 and [o for o, _ in seen] == sorted(o for o, _ in seen)  # last layer first, front of the arena
    assert sum(n for _, n in seen) == tr.arena_len
    assert all(seen[i][0] + seen[i][1] == seen[i + 1][0] for i in range(len(seen) - 1))
    tr.close()


def test_double_buffered_upload_matches_synchronous_steps(gpu):
    """The double-buffered upload path (wb_dp_submit: batch i+1 copied while step i runs, the trainer reading from the slot
    buffers) gives bit-identical losses to uploading each batch and stepping in turn."""
    import torch

    from weta_b200.trainer import DataParallelTrainer

    cfg = CnnConfig("tiny", 3, 8, 8, 16, 32)
    batch, steps = 32, 5
    host = []
    for s in range(steps):
        x, y = synthetic_batch(cfg, batch, s, 0, gpu)
        hx = torch.from_numpy(np.ascontiguousarray(x.numpy(), dtype=np.float32).reshape(-1)).pin_memory()
        hy = torch.from_numpy(np.ascontiguousarray(y.numpy(), dtype=np.int64).reshape(-1)).pin_memory()
        host.append((hx, hy))

    def run(prefetch):
        manual_seed(7)
        tr = FusedTrainer(gpu, cnn_specs(cfg), batch, (cfg.in_ch, cfg.hw, cfg.hw), lr=1e-3, matmul_mode=FP32)
        tr.init_from_global_rng()
        losses = []
        if prefetch:
            dp = DataParallelTrainer(tr, 0, 1, None)
            dp.submit(host[0][0].data_ptr(), host[0][1].data_ptr())
            for s in range(steps):
                if s + 1 < steps:
                    dp.submit(host[s + 1][0].data_ptr(), host[s + 1][1].data_ptr())
                losses.append(dp.step_submitted())
            dp.close()
        else:
            for s in range(steps):
                losses.append(tr.step_host(host[s][0].data_ptr(), host[s][1].data_ptr()))
        tr.close()
        return losses

    assert run(True) == run(False)


@pytest.mark.parametrize("model", ["mlp", "cnn"])
def test_step_replayed_from_a_graph_equals_the_launch_by_launch_step(gpu, model):
    """wb_trainer_step after wb_trainer_use_graph: the whole step is captured once and replayed with the dropout seeds and
    the Adam scalars of each step rewritten in the graph.  Same seeds, same batches: losses and every parameter must be
    bit-identical to forward_backward + adam_step issued launch by launch, over steps that straddle the capture."""
    from weta_b200.trainer import mlp_specs
    from weta_b200.workloads import MNIST_CNN

    if model == "mlp":
        specs, batch, shape = mlp_specs(), 128, (784, 1, 1)
    else:
        specs, batch, shape = cnn_specs(MNIST_CNN), 64, (1, 28, 28)
    rng = np.random.default_rng(5)
    xs = [rng.random((batch,) + shape, dtype=np.float32) for _ in range(6)]
    ys = [rng.integers(0, 10, batch).astype(np.int64) for _ in range(6)]
    out = {}
    for graph in (False, True):
        manual_seed(21)
        tr = FusedTrainer(gpu, specs, batch, shape, lr=1e-3, matmul_mode=TF32)
        tr.init_from_global_rng()
        tr.use_graph(graph)
        losses = []
        for x, y in zip(xs, ys):
            tr.stage(x, y)
            tr.step()
            losses.append(tr.loss())
        gpu.gemm_check()
        out[graph] = (losses, [tr.get_param(i) for i in range(len(tr.ranges))])
        tr.close()
    assert out[True][0] == out[False][0]
    for a, b in zip(out[True][1], out[False][1]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("model", ["mlp", "cnn", "wide"])
def test_programmatic_dependent_launch_changes_no_result(gpu, model):
    """The trainer's kernels are launched as programmatic dependents of the kernel before them (their launch overlaps that
    kernel's tail; each waits for it before touching memory).  Six steps with and without the attribute, in two child
    processes: every loss and every parameter bit for bit the same."""
    import json
    import os
    import subprocess
    import sys

    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "pdl_worker.py")
    out = {}
    for off in ("0", "1"):
        env = dict(os.environ, WETA_B200_NO_PDL=off)
        r = subprocess.run([sys.executable, worker, model], env=env, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        out[off] = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["0"]["losses"] == out["1"]["losses"]
    assert out["0"]["params"] == out["1"]["params"]


def test_graph_is_captured_again_when_the_staged_batch_moves(gpu):
    """The capture bakes in the address of the staged batch.  wb_trainer_set_input points the trainer at another
    device buffer: the next step must not replay the old graph on the old buffer."""
    specs, batch, shape = mlp_specs(), 64, (784, 1, 1)
    rng = np.random.default_rng(6)
    xs = [rng.random((batch, 784), dtype=np.float32) for _ in range(5)]
    ys = [rng.integers(0, 10, batch).astype(np.int64) for _ in range(5)]
    P = ctypes.c_void_p
    out = {}
    for graph in (False, True):
        manual_seed(3)
        tr = FusedTrainer(gpu, specs, batch, shape, lr=1e-3, matmul_mode=TF32)
        tr.init_from_global_rng()
        tr.use_graph(graph)
        # steps 0-2 on the trainer's own staging buffers, steps 3-4 on buffers the caller owns
        ext_x = Tensor.from_numpy(xs[3], gpu)
        ext_y = Tensor.from_numpy(ys[3], gpu)
        losses = []
        for i in range(5):
            if i < 3:
                tr.stage(xs[i], ys[i])
            elif i == 3:
                gpu.check(tr.lib.wb_trainer_set_input(tr.handle, P(ext_x.storage.ptr), P(ext_y.storage.ptr)))
            else:
                ext_x2, ext_y2 = Tensor.from_numpy(xs[4], gpu), Tensor.from_numpy(ys[4], gpu)
                gpu.check(tr.lib.wb_trainer_set_input(tr.handle, P(ext_x2.storage.ptr), P(ext_y2.storage.ptr)))
            tr.step()
            losses.append(tr.loss())
        out[graph] = (losses, [tr.get_param(i) for i in range(len(tr.ranges))])
        gpu.check(tr.lib.wb_trainer_set_input(tr.handle, None, None))
        tr.close()
    assert out[True][0] == out[False][0]
    for a, b in zip(out[True][1], out[False][1]):
        assert np.array_equal(a, b)
