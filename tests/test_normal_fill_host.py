"""CPU-only: the correctly rounded ln / cos behind the Normal fill (weta_b200/csrc/normal_dd.h, compiled for the host inside
the library) against arbitrary-precision values, and the whole sample against the oracle's libm-based one
(Distribution::sample, crates/weta-core/src/ops.rs:182-186)."""
import ctypes
import random

import numpy as np
import pytest

from oracle.mirror.tensor import Tensor
from weta_b200.backend import load_library
from weta_b200.core import Distribution, DType


def _lib():
    lib = load_library()
    lib.wb_host_log_rn.argtypes = [ctypes.c_double]
    lib.wb_host_log_rn.restype = ctypes.c_double
    lib.wb_host_cos_rn.argtypes = [ctypes.c_double]
    lib.wb_host_cos_rn.restype = ctypes.c_double
    lib.wb_host_normal_sample.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_double, ctypes.c_double]
    lib.wb_host_normal_sample.restype = ctypes.c_double
    return lib


def test_log_and_cos_are_correctly_rounded():
    mpmath = pytest.importorskip("mpmath")
    lib = _lib()
    mpmath.mp.prec = 200
    rnd = random.Random(1)
    ks = [0, 1, 2, (1 << 53) - 1, (1 << 53) - 2, 1 << 52, (1 << 52) + 1]          # u1 = 1, just below 1, 2^-53, 1/2 ...
    ks += [rnd.getrandbits(10) for _ in range(100)] + [(1 << 53) - 1 - rnd.getrandbits(12) for _ in range(100)]
    ks += [rnd.getrandbits(53) for _ in range(3000)]
    for k in ks:
        u1 = 1.0 - k * 2.0 ** -53
        assert lib.wb_host_log_rn(u1) == float(mpmath.log(mpmath.mpf(u1))), u1
    ts = [0.0, 6.283185307179586 * (1.0 - 2.0 ** -53), 1.5707963267948966, 3.141592653589793, 4.71238898038469, 0.7853981633974483]
    ts += [6.283185307179586 * (rnd.getrandbits(53) * 2.0 ** -53) for _ in range(3000)]
    # arguments a few ulp from the multiples of pi/2, where the reduction cancels most
    for base in (1.5707963267948966, 3.141592653589793, 4.71238898038469, 6.283185307179586):
        ts += [float(np.nextafter(base, 0.0)), float(np.nextafter(np.nextafter(base, 0.0), 0.0)), float(np.nextafter(base, 10.0))]
    for t in ts:
        if t < 8.0:
            assert lib.wb_host_cos_rn(t) == float(mpmath.cos(mpmath.mpf(t))), t


def test_normal_samples_against_the_oracle(oracle):
    """Against the oracle's libm evaluation: the f32 values agree exactly; in f64 the two may differ where libm's ln or
    cos is not correctly rounded (a fraction of a percent of elements), and then by a few units in the last place."""
    lib = _lib()
    n, seed = 1 << 15, 42
    mine = np.array([lib.wb_host_normal_sample(seed, i, 0.5, 2.0) for i in range(n)])
    theirs = Tensor.random_seeded([n], Distribution.normal(0.5, 2.0), DType.F64, oracle, seed).numpy()
    differ = mine != theirs
    assert differ.mean() < 0.01, differ.mean()
    # the sum mean + product can cancel, so the last place is that of the larger of its terms
    assert np.all(np.abs(mine - theirs) <= 8 * np.spacing(np.abs(theirs - 0.5) + 0.5))
    assert np.array_equal(mine.astype(np.float32), theirs.astype(np.float32))
