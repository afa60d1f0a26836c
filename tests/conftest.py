import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "matmul_golden.npz")
    z = np.load(path)
    cases = {}
    for key in z.files:
        name, dtype, field = key.split("/")
        cases.setdefault((name, dtype), {})[field] = z[key]
    return cases


@pytest.fixture(scope="session")
def linear_golden():
    import numpy as np
    z = np.load(os.path.join(ROOT, "tests", "golden", "linear_golden.npz"))
    cases = {}
    for key in z.files:
        name, dtype, field = key.split("/")
        cases.setdefault((name, dtype), {})[field] = z[key]
    return cases


@pytest.fixture(scope="session")
def lstm_gates_golden():
    import numpy as np
    z = np.load(os.path.join(ROOT, "tests", "golden", "lstm_gates_golden.npz"))
    cases = {}
    for key in z.files:
        name, dtype, field = key.split("/")
        cases.setdefault((name, dtype), {})[field] = z[key]
    return cases


def _load_cases(fname):
    import numpy as np
    z = np.load(os.path.join(ROOT, "tests", "golden", fname))
    cases = {}
    for key in z.files:
        name, dtype, field = key.split("/")
        cases.setdefault((name, dtype), {})[field] = z[key]
    return cases


@pytest.fixture(scope="session")
def gru_cell_golden():
    return _load_cases("gru_cell_golden.npz")


@pytest.fixture(scope="session")
def conv2d_golden():
    return _load_cases("conv2d_golden.npz")
