import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.cpu_backend import OracleBackend
    return OracleBackend()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "reference_fixture.npz")))


@pytest.fixture(scope="session")
def gpu():
    """The CUDA backend.  Fails loudly (never falls back) when the extension or device is missing."""
    from weta_b200.backend import B200Backend
    return B200Backend(0)


@pytest.fixture(scope="session")
def report():
    """report(name, **numbers): appends one JSON line of measured figures (actual error against the tolerance asserted,
    timings) to the file named by WETA_B200_TEST_REPORT, when that variable is set; otherwise does nothing."""
    import json

    path = os.environ.get("WETA_B200_TEST_REPORT")

    def write(name, **numbers):
        if path:
            with open(path, "a") as f:
                f.write(json.dumps({"test": name, **numbers}) + "\n")

    return write


# How tcgen05.mma kind::tf32 reads an f32 operand (1 = low 13 mantissa bits dropped, 2 / 3 = rounded to nearest); pinned
# on the GPU by tests/test_gpu_gemm.py::test_how_the_tensor_core_reads_an_f32_operand_as_tf32.
TF32_OPERAND_RULE = 1


@pytest.fixture()
def tf32_oracle(oracle):
    """The oracle with f32 matmul operands reduced to TF32 by that rule and the sum over k kept in double: what a TF32
    tensor-core contraction computes, up to the GPU's own accumulation error.  Restored to the plain restatement afterwards."""
    oracle.set_matmul_test_mode(TF32_OPERAND_RULE, True)
    try:
        yield oracle
    finally:
        oracle.set_matmul_test_mode(0, False)
