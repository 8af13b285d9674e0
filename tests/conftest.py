import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def own():
    import oracle
    return oracle.own()


@pytest.fixture(scope="session")
def ref():
    import oracle
    r = oracle.ref()
    if r is None:
        pytest.skip("oracle/_ref (the compiled reference CPU code) is not present here")
    return r


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    here = os.path.join(ROOT, "tests", "golden")
    return (np.load(os.path.join(here, "reference_cpu_vectors.npz")),
            np.load(os.path.join(here, "rope_hf_capture.npz")))
