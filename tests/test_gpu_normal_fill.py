"""The Normal fill of Backend::random on the GPU (crates/weta-core/src/ops.rs:182-186) against the CPU oracle, counted
element by element at the sizes the reference's RNG test never reaches (crates/weta/tests/cuda_parity.rs:150-165 asks
1e-6 on 1000 values)."""
import ctypes

import numpy as np
import pytest

from oracle.mirror.tensor import Tensor
from weta_b200.core import Distribution, DType

pytestmark = pytest.mark.gpu


def test_f32_normal_fill_2_pow_28_is_bit_identical(oracle, gpu, report):
    n, seed = 1 << 28, 42
    got = Tensor.random_seeded([n], Distribution.normal(0.0, 1.0), DType.F32, gpu, seed).numpy()
    want = Tensor.random_seeded([n], Distribution.normal(0.0, 1.0), DType.F32, oracle, seed).numpy()
    mismatches = int((got.view(np.uint32) != want.view(np.uint32)).sum())
    report("normal fill f32 2^28 seed 42", mismatches=mismatches)
    assert mismatches == 0


def test_f32_normal_fill_with_mean_and_std(oracle, gpu):
    for mean, std, seed, n in ((3.0, 0.25, 7, (1 << 22) + 3), (-1e3, 10.0, 8, 1 << 20)):
        got = Tensor.random_seeded([n], Distribution.normal(mean, std), DType.F32, gpu, seed).numpy()
        want = Tensor.random_seeded([n], Distribution.normal(mean, std), DType.F32, oracle, seed).numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (mean, std)


def test_f64_normal_fill_2_pow_24(oracle, gpu, report):
    """f64 fills equal the library's own host evaluation exactly (same source on both machines) and the oracle's libm
    evaluation wherever libm rounds ln and cos correctly: the honest count of the rest is reported and bounded."""
    n, seed = 1 << 24, 42
    got = Tensor.random_seeded([n], Distribution.normal(0.0, 1.0), DType.F64, gpu, seed).numpy()
    want = Tensor.random_seeded([n], Distribution.normal(0.0, 1.0), DType.F64, oracle, seed).numpy()
    differ = got != want
    worst = float((np.abs(got - want) / np.spacing(np.abs(want)))[differ].max()) if differ.any() else 0.0
    report("normal fill f64 2^24 seed 42", mismatches=int(differ.sum()), fraction=float(differ.mean()), worst_ulp=worst)
    assert differ.mean() < 0.01 and worst <= 8.0
    lib = gpu.lib
    lib.wb_host_normal_sample.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_double, ctypes.c_double]
    lib.wb_host_normal_sample.restype = ctypes.c_double
    idx = np.concatenate([np.arange(2048), np.flatnonzero(differ)[:2048], np.random.default_rng(0).integers(0, n, 2048)])
    host = np.array([lib.wb_host_normal_sample(seed, int(i), 0.0, 1.0) for i in idx])
    assert np.array_equal(host, got[idx])
