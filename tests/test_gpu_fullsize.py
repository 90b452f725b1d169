"""Parity at the sizes the micro-benchmarks time (fp32 N(0,1) data from the counter RNG): the kernels pick their
variants by size (slab splits of the per-channel reductions, 128-bit tile kernels for transposed views, CTA-pair and
two-row-block GEMM tiles), so the small cases of the other test files do not reach this code.  Element-wise ops on
[256,64,56,56] contiguous and as transposed views, BatchNorm2d forward / backward on the same tensor, softmax
cross-entropy on [8192,1000], matmul 4096^3 with both gradients, the convolution [64,32,14,14] * [64,32,3,3] + bias with
all its gradients, Adam on 10^8 parameters; each against the CPU oracle, which needs a few seconds per case."""
import ctypes

import numpy as np
import pytest

from oracle.mirror import nn
from oracle.mirror.autograd import Var
from oracle.mirror.tensor import Tensor, allclose
from weta_b200.core import Distribution, DType, Layout
from weta_b200.trainer import _declare

pytestmark = pytest.mark.gpu
SHAPE = [256, 64, 56, 56]
P = ctypes.c_void_p


def randn(shape, seed, be, dt=DType.F32):
    return Tensor.random_seeded(shape, Distribution.normal(0.0, 1.0), dt, be, seed)


@pytest.mark.parametrize("view", ["contiguous", "transpose(1,3)", "transpose(0,1)"])
def test_elementwise_on_256x64x56x56(oracle, gpu, view):
    """add, mul, relu forward and their backward products: exact IEEE operations, so the comparison is bit for bit."""
    mk = {"contiguous": lambda t: t, "transpose(1,3)": lambda t: t.transpose(1, 3), "transpose(0,1)": lambda t: t.transpose(0, 1)}[view]
    xs, ys = {}, {}
    for name, be in (("cpu", oracle), ("gpu", gpu)):
        x, y, g = mk(randn(SHAPE, 1, be)), mk(randn(SHAPE, 2, be)), mk(randn(SHAPE, 3, be))
        xs[name] = {"add": x.add(y), "mul": x.mul(y), "relu": x.relu(), "mul_bwd_a": g.mul(y), "relu_bwd": g.mul(x.step())}
    for k in xs["cpu"]:
        c, d = xs["cpu"][k].numpy(), xs["gpu"][k].numpy()
        assert c.shape == d.shape and np.array_equal(c, d), f"{k} on {view}: {int((c != d).sum())} elements differ"


def test_fused_relu_backward_on_256x64x56x56(oracle, gpu):
    _declare(gpu.lib)
    n = int(np.prod(SHAPE))
    want = randn(SHAPE, 3, oracle).mul(randn(SHAPE, 1, oracle).step()).numpy().reshape(-1)
    g, x = randn(SHAPE, 3, gpu), randn(SHAPE, 1, gpu)
    out = gpu.alloc(n, DType.F32)
    gpu.check(gpu.lib.wb_relu_bwd(gpu.handle, P(g.storage.ptr), P(x.storage.ptr), P(out.ptr), n))
    assert np.array_equal(gpu.to_host(out, Layout.contiguous([n]), DType.F32), want)


def test_batch_norm_2d_on_256x64x56x56(oracle, gpu, report):
    _declare(gpu.lib)
    n, c, h, w = SHAPE
    x, up = randn(SHAPE, 1, oracle), randn(SHAPE, 3, oracle)
    gamma, beta = randn([c], 4, oracle), randn([c], 5, oracle)
    xv, gv, bv = Var(x, requires_grad=True), Var(gamma, requires_grad=True), Var(beta, requires_grad=True)
    rm, rv = Tensor.zeros([c], DType.F32, oracle), Tensor.ones([c], DType.F32, oracle)
    y = nn.batch_norm(xv, rm, rv, gv, bv, True, 0.1, 1e-5)
    y.mul(Var(up)).sum().backward()
    lib, H = gpu.lib, gpu.handle
    xg, ug, gg, bg = randn(SHAPE, 1, gpu), randn(SHAPE, 3, gpu), randn([c], 4, gpu), randn([c], 5, gpu)
    rmg, rvg = Tensor.zeros([c], DType.F32, gpu), Tensor.ones([c], DType.F32, gpu)
    E = x.numel()
    ys, sm, sr = gpu.alloc(E, DType.F32), gpu.alloc(c, DType.F32), gpu.alloc(c, DType.F32)
    gpu.check(lib.wb_bn2d_fwd(H, P(xg.storage.ptr), n, c, h * w, P(gg.storage.ptr), P(bg.storage.ptr), P(rmg.storage.ptr), P(rvg.storage.ptr), 0.1, 1e-5,
                              P(ys.ptr), P(sm.ptr), P(sr.ptr)))
    got_y = gpu.to_host(ys, Layout.contiguous([E]), DType.F32).reshape(SHAPE)
    err_y = float(np.abs(got_y - y.numpy()).max())
    assert allclose(got_y, y.numpy(), 1e-5, 1e-5), err_y
    assert allclose(rmg.numpy(), rm.numpy(), 1e-5, 1e-6) and allclose(rvg.numpy(), rv.numpy(), 1e-5, 1e-6)
    dxs, dgs, dbs = gpu.alloc(E, DType.F32), gpu.alloc(c, DType.F32), gpu.alloc(c, DType.F32)
    gpu.check(lib.wb_bn2d_bwd(H, P(xg.storage.ptr), P(ug.storage.ptr), n, c, h * w, P(gg.storage.ptr), P(sm.ptr), P(sr.ptr), P(dxs.ptr), P(dgs.ptr),
                              P(dbs.ptr)))
    got_dx = gpu.to_host(dxs, Layout.contiguous([E]), DType.F32).reshape(SHAPE)
    got_dg, got_db = gpu.to_host(dgs, Layout.contiguous([c]), DType.F32), gpu.to_host(dbs, Layout.contiguous([c]), DType.F32)
    # The oracle adds 802 816 values per channel one after the other in f32; its own rounding is ~1e-4 of a sum's size.
    scale = float(np.abs(gv.grad.numpy()).max())
    report("BatchNorm2d [256,64,56,56]", y_max_err=err_y, dx_max_err=float(np.abs(got_dx - xv.grad.numpy()).max()),
           dgamma_rel_err=float(np.abs(got_dg - gv.grad.numpy()).max() / scale))
    assert allclose(got_dx, xv.grad.numpy(), 1e-4, 2e-5)
    assert np.abs(got_dg - gv.grad.numpy()).max() <= 3e-4 * scale
    assert np.abs(got_db - bv.grad.numpy()).max() <= 3e-4 * float(np.abs(bv.grad.numpy()).max())


def test_softmax_cross_entropy_on_8192x1000(oracle, gpu):
    _declare(gpu.lib)
    rows, cols = 8192, 1000
    z = randn([rows, cols], 10, oracle)
    lab = Tensor.random_seeded([rows], Distribution.uniform(0.0, float(cols)), DType.I64, oracle, 99)
    zv = Var(z, requires_grad=True)
    loss = zv.cross_entropy(lab)
    loss.backward()
    zg = randn([rows, cols], 10, gpu)
    lg = Tensor.random_seeded([rows], Distribution.uniform(0.0, float(cols)), DType.I64, gpu, 99)
    assert np.array_equal(lg.numpy(), lab.numpy())
    dz, ls, ps = gpu.alloc(rows * cols, DType.F32), gpu.alloc(1, DType.F32), gpu.alloc(rows * cols, DType.F32)
    gpu.check(gpu.lib.wb_softmax_ce(gpu.handle, P(zg.storage.ptr), P(lg.storage.ptr), rows, cols, P(ps.ptr), P(dz.ptr), None, P(ls.ptr), 1.0))
    got_loss = float(gpu.to_host(ls, Layout.contiguous([1]), DType.F32)[0])
    assert abs(got_loss - loss.item()) <= 1e-5 * abs(loss.item())
    assert allclose(gpu.to_host(dz, Layout.contiguous([rows, cols]), DType.F32).reshape(rows, cols), zv.grad.numpy(), 1e-4, 1e-9)
    assert allclose(gpu.to_host(ps, Layout.contiguous([rows, cols]), DType.F32).reshape(rows, cols), z.softmax(1).numpy(), 1e-4, 1e-8)


@pytest.mark.parametrize("mode", [1, 0])
def test_matmul_4096_cubed_forward_and_both_gradients(gpu, mode):
    """A.B, G.B^T and A^T.G (the operand layouts MatmulBw hands over, crates/weta-autograd/src/ops.rs:821-827) against
    float64 on 48 sampled rows and all columns of each product."""
    n = 4096
    a, b, g = randn([n, n], 1, gpu), randn([n, n], 2, gpu), randn([n, n], 3, gpu)
    an, bn, gn = (t.numpy().astype(np.float64) for t in (a, b, g))
    rows = np.random.default_rng(0).choice(n, 48, replace=False)
    rows[:3] = (0, 127, n - 1)
    gpu.set_matmul_mode(mode)
    try:
        cases = {"A.B": (a.matmul(b), an[rows] @ bn), "G.B^T": (g.matmul(b.t()), gn[rows] @ bn.T), "A^T.G": (a.t().matmul(g), an.T[rows] @ gn)}
        gpu.gemm_check()
    finally:
        gpu.set_matmul_mode(0)
    # one-product TF32: 10-bit operands, ~2.4e-4 relative per product over 4096 random-sign terms of size ~1;
    # 3xTF32: the f32 accumulator's truncation, about 2^-24 * K * |sum|
    tol = {1: 5e-3 * np.sqrt(n), 0: 2e-5 * np.sqrt(n) + 1.2e-7 * n * np.sqrt(n)}[mode]
    for name, (got, want) in cases.items():
        err = float(np.abs(got.numpy().astype(np.float64)[rows] - want).max())
        assert err <= tol, (name, mode, err, tol)


def test_convolution_64x32x14x14_with_bias_and_all_gradients(oracle, gpu, report):
    """[64,32,14,14] * [64,32,3,3], stride 1, padding 1, with bias: forward, dX, dW, db through the trait-call chain
    (im2col, matmul, add; MatmulBw, Im2ColBw, sums) on both backends, in the default 3xTF32 mode."""
    out = {}
    for name, be in (("cpu", oracle), ("gpu", gpu)):
        x = Var(randn([64, 32, 14, 14], 1, be), requires_grad=True)
        w = Var(randn([64, 32, 3, 3], 2, be), requires_grad=True)
        b = Var(randn([64], 3, be), requires_grad=True)
        y = nn.conv2d(x, w, b, stride=(1, 1), padding=(1, 1))
        y.mul(Var(randn([64, 64, 14, 14], 4, be))).sum().backward()
        out[name] = [y.numpy(), x.grad.numpy(), w.grad.numpy(), b.grad.numpy()]
    errs = {}
    for k, c, g in zip(("y", "dx", "dw", "db"), out["cpu"], out["gpu"]):
        errs[k] = float(np.abs(g - c).max() / np.abs(c).max())
        assert errs[k] <= 1e-4, (k, errs[k])  # the reference's own matmul tolerance (cuda_parity.rs:172-188)
    report("conv [64,32,14,14]*[64,32,3,3] trait chain, 3xTF32", rel_err=errs)
    gpu.gemm_check()


def test_adam_on_1e8_parameters_is_bit_identical(oracle, gpu):
    _declare(gpu.lib)
    n = 100_000_000
    th = Var(randn([n], 20, oracle), requires_grad=True)
    opt = nn.Adam([th], 1e-3)
    tg, gg = randn([n], 20, gpu), randn([n], 21, gpu)
    mg, vg = Tensor.zeros([n], DType.F32, gpu), Tensor.zeros([n], DType.F32, gpu)
    for t in (1, 2):
        th.grad = randn([n], 21, oracle)
        opt.step()
        gpu.check(gpu.lib.wb_adam_step(gpu.handle, P(tg.storage.ptr), P(gg.storage.ptr), P(mg.storage.ptr), P(vg.storage.ptr), n, t, 1e-3, 0.9, 0.999,
                                       1e-8, 0.0, 0, 1.0))
        assert np.array_equal(tg.numpy(), th.numpy()), f"step {t}"
