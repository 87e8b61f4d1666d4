import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "slow: a GPU test whose CPU checker side takes tens of seconds (full-size shapes)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "quant_golden.npz")
    return np.load(path)


@pytest.fixture(scope="session")
def greedy_golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "greedy_golden.npz"))
