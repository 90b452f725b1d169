"""The implicit-GEMM 3x3 convolution (wb_conv3x3_fwd / wb_conv3x3_bwd) against the CPU oracle running the
reference's own chain: im2col -> matmul -> add bias (crates/weta-nn/src/functional.rs:84-106) and its
backward (crates/weta-autograd/src/ops.rs:821-827, 865-868)."""
import numpy as np
import pytest

from weta_b200.core import DType, Im2ColParams, Layout
from oracle.mirror.tensor import Tensor
from weta_b200.trainer import _declare

pytestmark = pytest.mark.gpu
P3 = Im2ColParams((3, 3), (1, 1), (1, 1), (1, 1))
# (n, c, h, w, o): square and non-square images, pixel counts that are not multiples of the 32-pixel K block
# or the 128/256-pixel tile, output channels below / above / not a multiple of the 128-row tile.
SHAPES = [(3, 128, 8, 8, 32), (2, 128, 6, 12, 160), (2, 256, 16, 16, 64), (1, 128, 20, 20, 96), (5, 128, 4, 4, 128),
          (3, 128, 16, 16, 256), (2, 128, 32, 16, 32),  # 16-wide: the kernels whose taps share pixel copies
          # widths 4 / 8 / 16 / 32 with a multiple of 128 pixels: the input gradient that reads dY without shifted copies
          (2, 128, 32, 4, 32), (2, 128, 16, 8, 64), (1, 128, 8, 32, 32), (2, 128, 24, 16, 96)]


def oracle_chain(oracle, x, w, bias, dy):
    n, c, h, wd = x.shape
    o = w.shape[0]
    xo, wo, bo, go = (Tensor.from_numpy(a, oracle) for a in (x, w, bias, dy))
    y = xo.conv2d(wo, bo, 1, 1).numpy()
    cols = xo.im2col(P3)
    g3 = go.reshape([n, o, h * wd])
    dw = g3.matmul(cols.transpose(1, 2)).sum_dims([0]).numpy().reshape(o, c, 3, 3)
    dx = wo.reshape([o, c * 9]).t().matmul(g3).col2im(P3, (c, h, wd)).numpy()
    return y, dw, dx


def run_gpu(gpu, x, w, bias, dy):
    _declare(gpu.lib)
    n, c, h, wd = x.shape
    o = w.shape[0]
    keep = [Tensor.from_numpy(np.ascontiguousarray(a), gpu) for a in (x, w, bias, dy)]
    xp, wp, bp, gp = (t.storage.ptr for t in keep)
    ys, dxs, dws = gpu.alloc(n * o * h * wd, DType.F32), gpu.alloc(x.size, DType.F32), gpu.alloc(w.size, DType.F32)
    gpu.check(gpu.lib.wb_conv3x3_fwd(gpu.handle, xp, wp, bp, n, c, h, wd, o, ys.ptr))
    gpu.check(gpu.lib.wb_conv3x3_bwd(gpu.handle, xp, wp, gp, n, c, h, wd, o, dxs.ptr, dws.ptr))
    gpu.gemm_check()
    get = lambda s, shape: gpu.to_host(s, Layout.contiguous(list(shape)), DType.F32).reshape(shape)
    return get(ys, (n, o, h, wd)), get(dws, w.shape), get(dxs, x.shape)


@pytest.mark.parametrize("shape", SHAPES)
def test_small_integer_operands_are_exact(oracle, gpu, shape):
    """Integers in [-2, 2] are TF32 values and every partial sum stays below 2^24, so padding, tap order,
    tap flipping and the sum over the batch must reproduce the oracle bit for bit."""
    n, c, h, wd, o = shape
    rng = np.random.default_rng(sum(shape))
    x = rng.integers(-2, 3, (n, c, h, wd)).astype(np.float32)
    w = rng.integers(-2, 3, (o, c, 3, 3)).astype(np.float32)
    bias = rng.integers(-4, 5, (o,)).astype(np.float32)
    dy = rng.integers(-2, 3, (n, o, h, wd)).astype(np.float32)
    want = oracle_chain(oracle, x, w, bias, dy)
    got = run_gpu(gpu, x, w, bias, dy)
    for name, g, r in zip(("y", "dweight", "dx"), got, want):
        assert np.array_equal(g, r), f"{name}: {np.count_nonzero(g != r)} of {r.size} differ, max {np.abs(g - r).max()}"


@pytest.mark.parametrize("shape", SHAPES[:3])
def test_normal_operands_within_tf32_rounding(oracle, gpu, shape):
    """N(0,1) operands: each product carries two 2^-11 operand roundings, so the result's error in the
    2-norm stays below 2e-3 of its norm (measured ~7e-4)."""
    n, c, h, wd, o = shape
    rng = np.random.default_rng(11 + sum(shape))
    x = rng.standard_normal((n, c, h, wd)).astype(np.float32)
    w = rng.standard_normal((o, c, 3, 3)).astype(np.float32)
    bias = rng.standard_normal((o,)).astype(np.float32)
    dy = rng.standard_normal((n, o, h, wd)).astype(np.float32)
    want = oracle_chain(oracle, x, w, bias, dy)
    got = run_gpu(gpu, x, w, bias, dy)
    for name, g, r in zip(("y", "dweight", "dx"), got, want):
        assert np.linalg.norm(g - r) <= 2e-3 * np.linalg.norm(r), name


def test_shapes_outside_the_rules_are_refused(gpu):
    _declare(gpu.lib)
    s = gpu.alloc(1 << 16, DType.F32)
    for n, c, h, wd, o in ((1, 64, 8, 8, 32), (1, 128, 7, 7, 32), (1, 128, 8, 8, 24)):
        assert gpu.lib.wb_conv3x3_fwd(gpu.handle, s.ptr, s.ptr, None, n, c, h, wd, o, s.ptr) == 2  # WB_ERR_UNSUPPORTED


def test_full_size_layer_equals_the_trait_chain_on_the_gpu(gpu):
    """The wide CNN's second convolution at its full per-GPU size ([4096,128,16,16] -> 256 channels), integer-valued
    operands: the implicit GEMM must equal, bit for bit, im2col -> matmul -> add and its backward run through the
    trait ops on the same GPU (every partial sum is an integer below 2^24, so TF32 and f32 products are both exact)."""
    _declare(gpu.lib)
    n, c, h, wd, o = 4096, 128, 16, 16, 256
    rng = np.random.default_rng(5)
    # small images of integers generated on the host once and tiled over the batch with a per-image sign pattern
    base = rng.integers(-2, 3, (64, c, h, wd)).astype(np.float32)
    x = np.ascontiguousarray(np.tile(base, (n // 64, 1, 1, 1)) * np.where(np.arange(n) % 3 == 0, -1.0, 1.0).astype(np.float32)[:, None, None, None])
    w = rng.integers(-1, 2, (o, c, 3, 3)).astype(np.float32)
    bias = rng.integers(-4, 5, (o,)).astype(np.float32)
    gbase = rng.integers(-1, 2, (64, o, h, wd)).astype(np.float32)
    dy = np.ascontiguousarray(np.tile(gbase, (n // 64, 1, 1, 1)))
    xt, wt, bt, gt = (Tensor.from_numpy(a, gpu) for a in (x, w, bias, dy))
    ys, dxs, dws = gpu.alloc(n * o * h * wd, DType.F32), gpu.alloc(x.size, DType.F32), gpu.alloc(w.size, DType.F32)
    gpu.check(gpu.lib.wb_conv3x3_fwd(gpu.handle, xt.storage.ptr, wt.storage.ptr, bt.storage.ptr, n, c, h, wd, o, ys.ptr))
    gpu.check(gpu.lib.wb_conv3x3_bwd(gpu.handle, xt.storage.ptr, wt.storage.ptr, gt.storage.ptr, n, c, h, wd, o, dxs.ptr, dws.ptr))
    gpu.gemm_check()
    y_i = Tensor(ys, Layout.contiguous([n, o, h, wd]), DType.F32, gpu)
    dx_i = Tensor(dxs, Layout.contiguous([n, c, h, wd]), DType.F32, gpu)
    dw_i = Tensor(dws, Layout.contiguous([o, c, 3, 3]), DType.F32, gpu)
    # the trait chain (3xTF32 matmul by default), compared on the device: max |difference| must be exactly 0
    y_e = xt.conv2d(wt, bt, 1, 1)
    assert float(y_e.sub(y_i).abs().max().numpy()) == 0.0
    del y_e
    cols = xt.im2col(P3)
    g3 = gt.reshape([n, o, h * wd])
    dx_e = wt.reshape([o, c * 9]).t().matmul(g3).col2im(P3, (c, h, wd))
    assert float(dx_e.sub(dx_i).abs().max().numpy()) == 0.0
    del dx_e
    # weight gradient: sums reach 4096 * 256 = 2^20 products of magnitude <= 2: still exact in f32
    dw_e = g3.matmul(cols.transpose(1, 2)).sum_dims([0]).reshape([o, c, 3, 3])
    assert float(dw_e.sub(dw_i).abs().max().numpy()) == 0.0
