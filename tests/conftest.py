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
