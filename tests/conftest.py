import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "bare.metal_b200"), os.path.join(ROOT, "oracle"), os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def product():
    """The product library. Missing library = hard failure: GPU tests must never pass on a fallback."""
    import bmapi
    return bmapi.load_product()


@pytest.fixture(scope="session")
def port():
    import oracle_check
    return oracle_check.load_port()


@pytest.fixture(scope="session")
def goldens():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "torch_kernel_goldens.npz"))
