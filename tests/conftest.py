"""pytest configuration: the `gpu` marker, import paths and shared fixtures."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "fixtures.npz"))


@pytest.fixture(scope="session")
def hb():
    """The CUDA library, bound to device 0.  GPU tests only."""
    from hearth_b200 import api
    api.init(0)
    yield api
    # whatever the kernels recorded on the device and no test asked for: an expired bounded wait, or - in the
    # bounds-checked build - an index outside its buffer
    api.check_status()
