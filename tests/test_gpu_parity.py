"""GPU backend against the CPU oracle, case for case with crates/weta/tests/cuda_parity.rs and with
the tolerances that file accepts; integer, gather and uniform-RNG results must be identical."""
import numpy as np
import pytest

from weta_b200.core import BinaryOp as B, DType, Distribution, Im2ColParams, UnaryOp as U
from oracle.mirror.tensor import Tensor, allclose

pytestmark = pytest.mark.gpu

RNG = np.random.default_rng(0)


def rand(shape, dt=np.float32):
    return RNG.standard_normal(shape).astype(dt)


def pair(oracle, gpu, arr):
    return Tensor.from_numpy(arr, oracle), Tensor.from_numpy(arr, gpu)


def same(name, cpu: Tensor, dev: Tensor, tol: float):
    assert dev.backend.name == "b200", f"{name}: result not on the GPU"
    c, g = cpu.numpy(), dev.numpy()
    assert c.shape == g.shape and c.dtype == g.dtype, f"{name}: {c.shape}/{c.dtype} vs {g.shape}/{g.dtype}"
    if tol == 0.0:
        assert np.array_equal(c, g, equal_nan=True), f"{name}: {np.sum(c != g)} of {c.size} differ"
    else:
        assert allclose(g, c, tol, tol), f"{name}: max err {np.nanmax(np.abs(g.astype(np.float64) - c))}"


FLOAT_UNARY = [(U.NEG, 0, 0), (U.EXP, 0, 0), (U.ABS, 0, 0), (U.SIGN, 0, 0), (U.RELU, 0, 0), (U.STEP, 0, 0),
               (U.TANH, 0, 0), (U.SIGMOID, 0, 0), (U.ERF, 0, 0), (U.SIN, 0, 0), (U.COS, 0, 0), (U.AFFINE, 2.5, -1.0),
               (U.GT_SCALAR, 0.3, 0), (U.MAX_SCALAR, 0.1, 0), (U.MIN_SCALAR, -0.2, 0)]
EXACT_UNARY = {U.NEG, U.ABS, U.SIGN, U.RELU, U.STEP, U.AFFINE, U.GT_SCALAR, U.MAX_SCALAR, U.MIN_SCALAR, U.RECIP, U.SQRT}


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_unary_kernels(oracle, gpu, dt):  # cuda_parity.rs:37-73
    tol = 1e-5 if dt == np.float32 else 1e-12
    c, g = pair(oracle, gpu, rand((3, 5, 4), dt))
    c, g = c.transpose(0, 2), g.transpose(0, 2)  # strided input
    for op, p1, p2 in FLOAT_UNARY:
        same(U.NAMES[op], c.unary(op, p1, p2), g.unary(op, p1, p2), 0.0 if op in EXACT_UNARY else tol)
    pc, pg = c.abs().add_scalar(0.1), g.abs().add_scalar(0.1)
    for op, p1 in [(U.LOG, 0), (U.SQRT, 0), (U.RECIP, 0), (U.POWF, 1.7)]:
        same(U.NAMES[op], pc.unary(op, p1), pg.unary(op, p1), 0.0 if op in EXACT_UNARY else tol)


def test_unary_i64(oracle, gpu):  # cuda_parity.rs:69-72
    c, g = pair(oracle, gpu, np.array([-3, 0, 4, 7], dtype=np.int64))
    for op, p1, p2 in [(U.NEG, 0, 0), (U.ABS, 0, 0), (U.RELU, 0, 0), (U.AFFINE, 2.0, 1.0), (U.SIGN, 0, 0), (U.STEP, 0, 0),
                       (U.GT_SCALAR, 0.5, 0), (U.MAX_SCALAR, 1.0, 0), (U.MIN_SCALAR, 1.0, 0)]:
        same(U.NAMES[op], c.unary(op, p1, p2), g.unary(op, p1, p2), 0.0)
    with pytest.raises(RuntimeError):
        g.unary(U.EXP)  # "not supported for i64 tensors"


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_binary_kernels_with_broadcasting(oracle, gpu, dt):  # cuda_parity.rs:75-109
    tol = 1e-5 if dt == np.float32 else 1e-12
    ac, ag = pair(oracle, gpu, rand((4, 3, 5), dt))
    bc, bg = pair(oracle, gpu, rand((5, 3), dt))
    bc, bg = bc.t(), bg.t()
    cc, cg = pair(oracle, gpu, rand((4, 1, 1), dt))
    for op in [B.ADD, B.SUB, B.MUL, B.DIV, B.MAXIMUM, B.MINIMUM, B.EQ, B.NE, B.LT, B.LE, B.GT, B.GE]:
        same(B.NAMES[op], ac.binary(op, bc), ag.binary(op, bg), 0.0)
        same(B.NAMES[op], ac.binary(op, cc), ag.binary(op, cg), 0.0)
    same("pow", ac.abs().add_scalar(0.1).pow(bc.abs()), ag.abs().add_scalar(0.1).pow(bg.abs()), tol * 10)


def test_binary_i64(oracle, gpu):  # cuda_parity.rs:105-108, plus negative divisors (Euclidean)
    xc, xg = pair(oracle, gpu, np.array([7, -7, 3, -7, 7], dtype=np.int64))
    yc, yg = pair(oracle, gpu, np.array([2, 2, 3, -2, -2], dtype=np.int64))
    for op in [B.ADD, B.SUB, B.MUL, B.DIV, B.EQ, B.MAXIMUM, B.MINIMUM, B.LT, B.GE]:
        same(B.NAMES[op], xc.binary(op, yc), xg.binary(op, yg), 0.0)
    pc, pg = pair(oracle, gpu, np.array([0, 1, 2, 3, 5], dtype=np.int64))
    same("pow", xc.pow(pc), xg.pow(pg), 0.0)


def test_nan_and_tie_rules(oracle, gpu):  # crates/weta-core/src/dtype.rs:136-149; weta-cpu/src/lib.rs:268-277
    a = np.array([[1.0, np.nan, 3.0, 3.0], [np.nan, 2.0, 2.0, -1.0], [0.0, -0.0, 5.0, 5.0]], dtype=np.float32)
    b = np.array([[np.nan, 1.0, 3.0, 4.0], [1.0, np.nan, 1.0, np.nan], [-0.0, 0.0, 5.0, 6.0]], dtype=np.float32)
    ac, ag = pair(oracle, gpu, a)
    bc, bg = pair(oracle, gpu, b)
    for op in [B.MAXIMUM, B.MINIMUM]:
        same(B.NAMES[op], ac.binary(op, bc), ag.binary(op, bg), 0.0)
    for d in (0, 1):
        same("max", ac.max_dims([d]), ag.max_dims([d]), 0.0)
        same("min", ac.min_dims([d]), ag.min_dims([d]), 0.0)
        same("argmax", ac.argmax(d), ag.argmax(d), 0.0)
        same("argmin", ac.argmin(d), ag.argmin(d), 0.0)
    long = np.zeros((3, 2000), dtype=np.float32)
    long[0, 7] = long[0, 1500] = 9.0   # tie: first wins
    long[1, 0] = np.nan                # NaN first: index 0
    long[2, 5] = np.nan                # NaN later never wins
    long[2, 1999] = 1.0
    lc, lg = pair(oracle, gpu, long)
    same("argmax long", lc.argmax(1), lg.argmax(1), 0.0)
    same("argmin long", lc.argmin(1), lg.argmin(1), 0.0)
    same("max long", lc.max_dims([1]), lg.max_dims([1]), 0.0)


def test_reductions(oracle, gpu):  # cuda_parity.rs:111-129
    c, g = pair(oracle, gpu, rand((6, 7, 8), np.float64))
    c, g = c.permute([2, 0, 1]), g.permute([2, 0, 1])
    for d in range(3):
        same("sum", c.sum_dims([d]), g.sum_dims([d]), 1e-12)
        same("max", c.max_dims([d], True), g.max_dims([d], True), 0.0)
        same("min", c.min_dims([d]), g.min_dims([d]), 0.0)
        same("argmax", c.argmax(d), g.argmax(d), 0.0)
        same("argmin", c.argmin(d), g.argmin(d), 0.0)
    same("sum all", c.sum(), g.sum(), 1e-12)
    same("softmax", c.softmax(1), g.softmax(1), 1e-12)
    ic, ig = pair(oracle, gpu, np.array([[3, 1, 4], [1, 5, 9]], dtype=np.int64))
    same("i64 sum", ic.sum_dims([1]), ig.sum_dims([1]), 0.0)
    same("i64 max", ic.max_dims([0]), ig.max_dims([0]), 0.0)


def test_long_axis_block_reductions(oracle, gpu):  # cuda_parity.rs:131-148
    for shape in [(3, 1000), (700, 5)]:
        c, g = pair(oracle, gpu, rand(shape, np.float64))
        for d in range(2):
            same("sum", c.sum_dims([d]), g.sum_dims([d]), 1e-10)
            same("max", c.max_dims([d]), g.max_dims([d]), 0.0)
            same("min", c.min_dims([d]), g.min_dims([d]), 0.0)
    c, g = pair(oracle, gpu, rand((64, 32, 28, 28)))
    c, g = c.permute([1, 0, 2, 3]), g.permute([1, 0, 2, 3])
    same("batch-norm style mean", c.mean_dims([1, 2, 3]), g.mean_dims([1, 2, 3]), 1e-4)


def test_reduce_kernel_variants(oracle, gpu):
    """Shapes that reach each reduction kernel: staged rows, column walk (with and without the split
    into scratch partials), block per output (single huge row split across blocks), generic."""
    cases = [((4096, 56), 1), ((300, 1000), 1), ((8192, 10), 0), ((50000, 64), 0), ((3, 70000), 1), ((1, 1 << 20), 1),
             ((37, 5, 11), 1), ((128, 64, 14), 2), ((128, 64), 0)]
    for shape, axis in cases:
        c, g = pair(oracle, gpu, rand(shape))
        same(f"sum {shape}/{axis}", c.sum_dims([axis]), g.sum_dims([axis]), 2e-4)
        same(f"max {shape}/{axis}", c.max_dims([axis]), g.max_dims([axis]), 0.0)
        same(f"argmin {shape}/{axis}", c.argmin(axis), g.argmin(axis), 0.0)
    # staged rows and the un-split column walk add in the CPU's order: sums are bit-identical
    for shape, axis in [((4096, 56), 1), ((128, 64), 0), ((2048, 1000), 1)]:
        c, g = pair(oracle, gpu, rand(shape))
        same(f"exact sum {shape}", c.sum_dims([axis]), g.sum_dims([axis]), 0.0)


@pytest.mark.parametrize("dt", [DType.F32, DType.F64])
def test_random_numbers_match_the_cpu_for_the_same_seed(oracle, gpu, dt):  # cuda_parity.rs:150-165
    for dist, shape, tol in [(Distribution.normal(0.0, 1.0), [10, 100], 1e-6), (Distribution.uniform(-2.0, 5.0), [3, 7], 0.0),
                             (Distribution.uniform(0.0, 1.0), [1000, 33], 0.0)]:
        same(str(dist), Tensor.random_seeded(shape, dist, dt, oracle, 9), Tensor.random_seeded(shape, dist, dt, gpu, 9), tol)
    labels_c = Tensor.random_seeded([4096], Distribution.uniform(0.0, 10.0), DType.I64, oracle, 20000)
    labels_g = Tensor.random_seeded([4096], Distribution.uniform(0.0, 10.0), DType.I64, gpu, 20000)
    same("integer draw", labels_c, labels_g, 0.0)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_matmul_layouts(oracle, gpu, dt):  # cuda_parity.rs:167-189
    tol = 1e-4 if dt == np.float32 else 1e-11
    T = lambda a: pair(oracle, gpu, a)
    cases = [
        (T(rand((5, 7), dt)), T(rand((7, 3), dt)), lambda a: a, lambda b: b),
        (T(rand((7, 5), dt)), T(rand((7, 3), dt)), lambda a: a.t(), lambda b: b),
        (T(rand((5, 7), dt)), T(rand((3, 7), dt)), lambda a: a, lambda b: b.t()),
        (T(rand((7, 5), dt)), T(rand((3, 7), dt)), lambda a: a.t(), lambda b: b.t()),
        (T(rand((2, 4, 5, 7), dt)), T(rand((7, 3), dt)), lambda a: a, lambda b: b),       # broadcast batch
        (T(rand((4, 1, 5, 7), dt)), T(rand((2, 7, 3), dt)), lambda a: a, lambda b: b),    # both broadcast
        (T(rand((1, 7), dt)), T(rand((7, 1), dt)), lambda a: a, lambda b: b),             # degenerate dims
        (T(rand((5, 14), dt)), T(rand((7, 3), dt)), lambda a: a.step_by(1, 2), lambda b: b),  # strided by 2
        (T(rand((7,), dt)), T(rand((7, 3), dt)), lambda a: a, lambda b: b),
    ]
    for i, ((ac, ag), (bc, bg), fa, fb) in enumerate(cases):
        same(f"matmul case {i}", fa(ac).matmul(fb(bc)), fa(ag).matmul(fb(bg)), tol)


def test_im2col_col2im_cast_copy(oracle, gpu):  # cuda_parity.rs:191-212
    xc, xg = pair(oracle, gpu, rand((2, 3, 7, 6)))
    p = Im2ColParams((3, 2), (2, 1), (1, 1), (1, 2))
    cols_c, cols_g = xc.im2col(p), xg.im2col(p)
    same("im2col", cols_c, cols_g, 0.0)
    same("im2col strided", xc.transpose(2, 3).im2col(p), xg.transpose(2, 3).im2col(p), 0.0)
    same("col2im", cols_c.col2im(p, (3, 7, 6)), cols_g.col2im(p, (3, 7, 6)), 0.0)
    p3 = Im2ColParams((3, 3), (1, 1), (1, 1), (1, 1))
    same("col2im 3x3", xc.im2col(p3).col2im(p3, (3, 7, 6)), xg.im2col(p3).col2im(p3, (3, 7, 6)), 0.0)
    for dt in (DType.F32, DType.F64, DType.I64):
        same("cast", xc.to_dtype(dt), xg.to_dtype(dt), 0.0)
    big = np.array([1.9, -1.9, np.nan, 1e30, -1e30, 2.0**63, -(2.0**63)], dtype=np.float64)
    bc, bg = pair(oracle, gpu, big)
    same("saturating cast", bc.to_dtype(DType.I64), bg.to_dtype(DType.I64), 0.0)
    ac, ag = pair(oracle, gpu, rand((2, 3)))
    bc, bg = pair(oracle, gpu, rand((4, 3)))
    same("cat", Tensor.cat([ac, bc], 0), Tensor.cat([ag, bg], 0), 0.0)
    ac.narrow(1, 1, 1).fill_(5.0)
    ag.narrow(1, 1, 1).fill_(5.0)
    same("in-place slice", ac, ag, 0.0)


def test_elementwise_layout_paths(oracle, gpu):
    """Every element-wise kernel: flat vectorised (with a ragged tail and an unaligned base), the
    strided path with broadcasts, and the shared-memory tile path for transposed views."""
    xc, xg = pair(oracle, gpu, rand((8, 6, 20, 24)))
    yc, yg = pair(oracle, gpu, rand((8, 6, 20, 24)))
    same("flat add", xc.add(yc), xg.add(yg), 0.0)
    same("tile relu (1,3)", xc.transpose(1, 3).relu(), xg.transpose(1, 3).relu(), 0.0)
    same("tile mul both transposed", xc.transpose(1, 3).mul(yc.transpose(1, 3)), xg.transpose(1, 3).mul(yg.transpose(1, 3)), 0.0)
    same("tile add mixed", xc.transpose(2, 3).add(yc.reshape([8, 6, 24, 20])), xg.transpose(2, 3).add(yg.reshape([8, 6, 24, 20])), 0.0)
    same("strided (0,1)", xc.transpose(0, 1).step(), xg.transpose(0, 1).step(), 0.0)
    chc, chg = pair(oracle, gpu, rand((1, 6, 1, 1)))
    same("channel broadcast", xc.mul(chc), xg.mul(chg), 0.0)
    rowc, rowg = pair(oracle, gpu, rand((24,)))
    same("row broadcast", xc.sub(rowc), xg.sub(rowg), 0.0)
    sc, sg = pair(oracle, gpu, rand(()))
    same("scalar broadcast", xc.mul(sc), xg.mul(sg), 0.0)
    same("narrow (odd offset)", xc.narrow(3, 1, 21).neg(), xg.narrow(3, 1, 21).neg(), 0.0)
    fc, fg = pair(oracle, gpu, rand((10007,)))
    same("ragged tail", fc.affine(3.0, 1.0), fg.affine(3.0, 1.0), 0.0)
    same("unaligned base", fc.narrow(0, 3, 10001).abs(), fg.narrow(0, 3, 10001).abs(), 0.0)
    same("every other", fc.step_by(0, 2).relu(), fg.step_by(0, 2).relu(), 0.0)
    ec, eg = pair(oracle, gpu, np.zeros((0, 5), dtype=np.float32))
    same("empty", ec.exp(), eg.exp(), 0.0)
    same("empty reduce", ec.sum_dims([0]), eg.sum_dims([0]), 0.0)
    dc, dg = pair(oracle, gpu, rand((5, 4, 3, 2, 3, 2, 2, 2), np.float64))
    perm = [7, 0, 6, 1, 5, 2, 4, 3]
    same("8-d permute", dc.permute(perm).tanh(), dg.permute(perm).tanh(), 1e-12)
