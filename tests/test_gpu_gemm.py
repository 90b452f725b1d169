"""The tcgen05 TF32 GEMM against float64 numpy: every operand layout the trait can hand over
(row-major, transposed, batched, batch-broadcast), ragged edges, split-K (two launches, and inside a cluster), 1x and
3x TF32."""
import numpy as np
import pytest

from oracle.mirror.tensor import Tensor

pytestmark = pytest.mark.gpu

TF32X3, TF32, FP32 = 0, 1, 2
RNG = np.random.default_rng(1)


def rnd(*shape):
    return RNG.standard_normal(shape).astype(np.float32)


def check(gpu, a_np, b_np, fa, fb, mode, name):
    gpu.set_matmul_mode(mode)
    a, b = fa(Tensor.from_numpy(a_np, gpu)), fb(Tensor.from_numpy(b_np, gpu))
    got = a.matmul(b).numpy().astype(np.float64)
    gpu.gemm_check()
    an = fa(_NP(a_np)).arr.astype(np.float64)
    bn = fb(_NP(b_np)).arr.astype(np.float64)
    want = an @ bn
    k = an.shape[-1]
    # Operands are N(0,1).  TF32 keeps 10 mantissa bits (the tensor core drops the rest), so one product
    # is off by up to ~2e-3 relative and a K-term sum by a few 1e-3*sqrt(K) at the worst output; 3xTF32
    # leaves the lo*lo term and the second truncation of lo: ~1e-6 relative per product.
    # The tensor core adds into its f32 accumulator with truncation, which leaves a bias of about
    # 2^-24 * K * |sum| (|sum| ~ sqrt(K) here); that term is what bounds 3xTF32 for long contractions.
    tol = {TF32: 5e-3, TF32X3: 2e-5, FP32: 3e-6}[mode] * np.sqrt(k) + 1.2e-7 * k * np.sqrt(k)
    err = np.abs(got - want).max()
    assert got.shape == want.shape, name
    assert err <= tol, f"{name} mode {mode}: max err {err:.3e} > {tol:.3e}"
    gpu.set_matmul_mode(TF32X3)


class _NP:
    """numpy stand-in with the view methods used by the cases below."""

    def __init__(self, arr):
        self.arr = arr

    def t(self):
        return _NP(np.swapaxes(self.arr, -1, -2))

    def step_by(self, dim, step):
        idx = [slice(None)] * self.arr.ndim
        idx[dim] = slice(None, None, step)
        return _NP(self.arr[tuple(idx)])

    def narrow(self, dim, start, length):
        idx = [slice(None)] * self.arr.ndim
        idx[dim] = slice(start, start + length)
        return _NP(self.arr[tuple(idx)])


ident = lambda x: x
tr = lambda x: x.t()


@pytest.mark.parametrize("mode", [TF32, TF32X3])
def test_operand_layouts(gpu, mode):
    m, n, k = 256, 384, 512
    check(gpu, rnd(m, k), rnd(k, n), ident, ident, mode, "NN (A K-major, B N-major)")
    check(gpu, rnd(m, k), rnd(n, k), ident, tr, mode, "NT (both K-major)")
    check(gpu, rnd(k, m), rnd(k, n), tr, ident, mode, "TN (both MN-major)")
    check(gpu, rnd(k, m), rnd(n, k), tr, tr, mode, "TT (A M-major, B K-major)")


@pytest.mark.parametrize("mode", [TF32, TF32X3])
def test_ragged_edges_and_small_k(gpu, mode):
    for m, n, k in [(200, 136, 100), (129, 127, 36), (1000, 12, 260), (128, 128, 32), (130, 260, 1028)]:
        check(gpu, rnd(m, k), rnd(k, n), ident, ident, mode, f"NN {m}x{n}x{k}")
        check(gpu, rnd(m, k), rnd(n, k), ident, tr, mode, f"NT {m}x{n}x{k}")
        check(gpu, rnd(k, m), rnd(k, n), tr, ident, mode, f"TN {m}x{n}x{k}")


@pytest.mark.parametrize("mode", [TF32, TF32X3])
def test_batched_and_broadcast(gpu, mode):
    check(gpu, rnd(6, 128, 96), rnd(6, 96, 192), ident, ident, mode, "batched")
    check(gpu, rnd(64, 288), rnd(5, 288, 196), ident, ident, mode, "weight broadcast over the batch (conv forward)")
    check(gpu, rnd(5, 64, 196), rnd(5, 288, 196), ident, tr, mode, "batched NT (conv weight gradient)")
    check(gpu, rnd(64, 288), rnd(5, 64, 196), tr, ident, mode, "broadcast transposed weight (conv input gradient)")


@pytest.mark.parametrize("mode", [TF32, TF32X3])
def test_split_k(gpu, mode):
    check(gpu, rnd(4096, 128), rnd(4096, 256), tr, ident, mode, "long K, few tiles (a weight gradient)")
    check(gpu, rnd(128, 8192), rnd(8192, 128), ident, ident, mode, "one tile, K = 8192")


@pytest.mark.parametrize("mode", [TF32, TF32X3])
def test_split_k_inside_a_cluster(gpu, mode):
    """Few 128 x 128 tiles and a short contraction: the K blocks are split over a cluster of 2, 4 or 8 CTAs that sum
    their partial tiles through distributed shared memory.  Whole and ragged tiles, every operand layout, a batch, and
    the same answer bit for bit on a second run."""
    for m, n, k in [(128, 128, 128), (128, 128, 256), (128, 128, 512), (100, 70, 520), (256, 256, 128), (130, 260, 1028 if mode == TF32 else 516),
                    (128, 512, 784), (37, 10 * 4, 2048 if mode == TF32 else 672)]:
        check(gpu, rnd(m, k), rnd(k, n), ident, ident, mode, f"NN {m}x{n}x{k}")
        check(gpu, rnd(m, k), rnd(n, k), ident, tr, mode, f"NT {m}x{n}x{k}")
        check(gpu, rnd(k, m), rnd(k, n), tr, ident, mode, f"TN {m}x{n}x{k}")
        check(gpu, rnd(k, m), rnd(n, k), tr, tr, mode, f"TT {m}x{n}x{k}")
    check(gpu, rnd(3, 128, 192), rnd(3, 192, 256), ident, ident, mode, "batched, three clusters per tile column")
    gpu.set_matmul_mode(mode)
    a, b = Tensor.from_numpy(rnd(200, 512), gpu), Tensor.from_numpy(rnd(512, 136), gpu)
    first, second = a.matmul(b).numpy(), a.matmul(b).numpy()
    gpu.gemm_check()
    gpu.set_matmul_mode(TF32X3)
    assert np.array_equal(first, second)


def test_fallback_layouts(gpu):
    """Operands TMA cannot describe go to the CUDA-core tiles and still give the right answer."""
    check(gpu, rnd(64, 130), rnd(65, 70), lambda a: a.step_by(1, 2), ident, TF32X3, "strided by 2")
    check(gpu, rnd(70, 67), rnd(67, 33), ident, ident, TF32X3, "pitch not a multiple of 4")
    check(gpu, rnd(512, 516), rnd(512, 256), lambda a: a.narrow(1, 1, 512), ident, TF32X3, "unaligned base")
    check(gpu, rnd(256, 256), rnd(256, 256), ident, ident, FP32, "fp32 mode")


def test_large_square(gpu):
    check(gpu, rnd(2048, 2048), rnd(2048, 2048), ident, ident, TF32, "2048^3 tf32")
    check(gpu, rnd(2048, 2048), rnd(2048, 2048), ident, tr, TF32X3, "2048^3 3xtf32 NT")


def test_how_the_tensor_core_reads_an_f32_operand_as_tf32(gpu, oracle, report):
    """TF32 keeps 10 mantissa bits.  Operands whose dropped 13 bits are 0.75, exactly 0.5 and just below 0.5 of a TF32
    step tell truncation from rounding to nearest: the rule found here is the one the oracle's TF32 test mode
    (conftest fixture `tf32_oracle`) must apply, or the tight fused-step tolerances would compare different operands."""
    cases = {"0.75": 1.0 + 2.0 ** -11 + 2.0 ** -12, "0.5": 1.0 + 2.0 ** -11, "0.49": 1.0 + 2.0 ** -11 - 2.0 ** -23,
             "-0.75": -(1.0 + 2.0 ** -11 + 2.0 ** -12), "odd+0.5": 1.0 + 2.0 ** -10 + 2.0 ** -11}
    b = np.zeros((32, 128), np.float32)
    b[0, :] = 1.0
    seen = {}
    gpu.set_matmul_mode(TF32)
    for name, a in cases.items():
        got = Tensor.from_numpy(np.full((128, 32), a, np.float32), gpu).matmul(Tensor.from_numpy(b, gpu)).numpy()
        assert np.all(got == got[0, 0])
        seen[name] = float(got[0, 0])
    gpu.gemm_check()
    gpu.set_matmul_mode(TF32X3)
    step = 2.0 ** -10
    rule = {(1.0, 1.0, 1.0, -1.0, 1.0 + step): 1,                           # low bits dropped
            (1.0 + step, 1.0 + step, 1.0, -(1.0 + step), 1.0 + 2 * step): 2,  # nearest, ties away from zero
            (1.0 + step, 1.0, 1.0, -(1.0 + step), 1.0 + 2 * step): 3}.get(   # nearest, ties to even
        (seen["0.75"], seen["0.5"], seen["0.49"], seen["-0.75"], seen["odd+0.5"]))
    report("tf32 operand read", seen=seen, rule=rule)
    from conftest import TF32_OPERAND_RULE
    assert rule == TF32_OPERAND_RULE, (seen, rule)
    # the oracle's test mode applies the same rule
    oracle.set_matmul_test_mode(TF32_OPERAND_RULE, True)
    try:
        for name, a in cases.items():
            want = Tensor.from_numpy(np.full((4, 32), a, np.float32), oracle).matmul(Tensor.from_numpy(b, oracle)).numpy()
            assert float(want[0, 0]) == seen[name], name
    finally:
        oracle.set_matmul_test_mode(0, False)


def test_a_pipeline_wait_that_runs_out_is_reported_and_the_context_survives(gpu):
    """The tensor-core kernels bound every mbarrier wait; when one runs out they raise a flag that wb_gemm_check turns
    into WB_ERR_TIMEOUT.  A one-thread kernel makes the same wait run out on a barrier nothing arrives at."""
    import ctypes

    from weta_b200.backend import BackendError

    lib = gpu.lib
    lib.wb_gemm_selftest_timeout.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.wb_gemm_selftest_timeout.restype = ctypes.c_int
    gpu.gemm_check()  # clean before
    gpu.check(lib.wb_gemm_selftest_timeout(gpu.handle, 4096))
    with pytest.raises(BackendError) as e:
        gpu.gemm_check()
    assert e.value.status == 6  # WB_ERR_TIMEOUT
    gpu.gemm_check()  # the flag was cleared
    a = Tensor.from_numpy(np.eye(64, dtype=np.float32), gpu)
    assert np.array_equal(a.matmul(a).numpy(), np.eye(64, dtype=np.float32))
    gpu.gemm_check()
