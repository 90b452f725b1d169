"""Extension entry points for linear, max-pool and ReLU backward against the CPU oracle running the reference's
definitions (crates/weta-nn/src/functional.rs:54-60, 121-130; crates/weta-autograd/src/ops.rs:85, 305-314, 821-827)."""
import numpy as np
import pytest

from oracle.mirror import nn
from oracle.mirror.autograd import Var
from weta_b200.core import DType, Layout
from oracle.mirror.tensor import Tensor, allclose
from weta_b200.trainer import _declare

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(23)


def up(gpu, arr):
    t = Tensor.from_numpy(np.ascontiguousarray(arr), gpu)
    return t, t.storage.ptr


def down(gpu, storage, shape):
    return gpu.to_host(storage, Layout.contiguous(list(shape)), DType.F32).reshape(shape)


@pytest.mark.parametrize("mode,tol", [(2, 1e-5), (0, 1e-5), (1, 2e-3)])  # FP32, 3xTF32, TF32
@pytest.mark.parametrize("shape", [(128, 784, 512), (37, 100, 10), (256, 256, 384)])
def test_linear_forward_backward(oracle, gpu, mode, tol, shape):
    _declare(gpu.lib)
    n, fin, fout = shape
    x = RNG.standard_normal((n, fin)).astype(np.float32)
    w = (RNG.standard_normal((fout, fin)) / np.sqrt(fin)).astype(np.float32)
    b = RNG.standard_normal(fout).astype(np.float32)
    g = RNG.standard_normal((n, fout)).astype(np.float32)
    xo, wo, bo = (Var(Tensor.from_numpy(a, oracle), requires_grad=True) for a in (x, w, b))
    yo = nn.linear(xo, wo, bo).relu()
    yo.mul(Var(Tensor.from_numpy(g, oracle))).sum().backward()
    gpu.set_matmul_mode(mode)
    try:
        keep = [up(gpu, a) for a in (x, w, b, g)]
        (_, xp), (_, wp), (_, bp), (_, gp) = keep
        ys, dxs, dws, dbs, gzs = (gpu.alloc(k, DType.F32) for k in (n * fout, x.size, w.size, fout, n * fout))
        gpu.check(gpu.lib.wb_linear_fwd(gpu.handle, xp, wp, bp, n, fin, fout, 1, ys.ptr))
        gpu.check(gpu.lib.wb_relu_bwd(gpu.handle, gp, ys.ptr, gzs.ptr, n * fout))
        gpu.check(gpu.lib.wb_linear_bwd(gpu.handle, xp, wp, gzs.ptr, n, fin, fout, dxs.ptr, dws.ptr, dbs.ptr))
        gpu.gemm_check()
    finally:
        gpu.set_matmul_mode(0)
    scale = lambda a: tol * max(1.0, float(np.abs(a).max()))
    assert np.abs(down(gpu, ys, (n, fout)) - yo.data.numpy()).max() <= scale(yo.data.numpy())
    if mode == 1:
        # TF32 forward values near zero flip a few ReLU gates; compare the gradients in the 2-norm
        close = lambda a, r: np.linalg.norm(a - r) <= 2e-2 * np.linalg.norm(r)
    else:
        close = lambda a, r: np.abs(a - r).max() <= 10 * scale(r)
    assert close(down(gpu, dws, w.shape), wo.grad.numpy())
    assert close(down(gpu, dbs, (fout,)), bo.grad.numpy())
    assert close(down(gpu, dxs, x.shape), xo.grad.numpy())


@pytest.mark.parametrize("geom", [(6, 8, 12, 2, 2), (5, 9, 9, 3, 2), (4, 7, 10, 3, 1), (3, 4, 4, 2, 2)])
def test_max_pool_with_ties_is_exact(oracle, gpu, geom):
    """Values drawn from a few levels so windows tie; forward is exact, backward equals the oracle's mask/count
    route (non-overlapping windows exactly, overlapping ones up to the order of a few additions)."""
    _declare(gpu.lib)
    planes, h, w, k, s = geom
    x = RNG.integers(-2, 3, (1, planes, h, w)).astype(np.float32)
    oh, ow = (h - k) // s + 1, (w - k) // s + 1
    g = RNG.standard_normal((1, planes, oh, ow)).astype(np.float32)
    xo = Var(Tensor.from_numpy(x, oracle), requires_grad=True)
    yo = nn.max_pool2d(xo, k, s)
    yo.mul(Var(Tensor.from_numpy(g, oracle))).sum().backward()
    (xt, xp), (gt, gp) = up(gpu, x), up(gpu, g)  # the tensors own the device blocks: keep them alive
    ys, dxs = gpu.alloc(planes * oh * ow, DType.F32), gpu.alloc(x.size, DType.F32)
    gpu.check(gpu.lib.wb_maxpool2d_fwd(gpu.handle, xp, planes, h, w, k, s, ys.ptr))
    gpu.check(gpu.lib.wb_maxpool2d_bwd(gpu.handle, xp, gp, planes, h, w, k, s, dxs.ptr))
    assert np.array_equal(down(gpu, ys, (1, planes, oh, ow)), yo.data.numpy())
    got, want = down(gpu, dxs, x.shape), xo.grad.numpy()
    if s >= k:
        assert np.array_equal(got, want)
    else:
        assert allclose(got, want, 1e-6, 1e-6)


def test_max_pool_nan_wins(gpu):
    _declare(gpu.lib)
    x = np.array([[1.0, np.nan], [3.0, 2.0]], np.float32).reshape(1, 2, 2)
    xt, xp = up(gpu, x)
    ys = gpu.alloc(1, DType.F32)
    gpu.check(gpu.lib.wb_maxpool2d_fwd(gpu.handle, xp, 1, 2, 2, 2, 2, ys.ptr))
    assert np.isnan(down(gpu, ys, (1,))[0])
