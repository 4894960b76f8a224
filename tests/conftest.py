import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def native_lib():
    """The built C-ABI library (compiled on demand; nvcc needs no GPU)."""
    from flagdnn_b200 import _native, build

    build.build()
    return _native.load()


@pytest.fixture(scope="session")
def golden_next():
    """Outputs of the unmodified reference (CPU graphs) for the rows next to the path: block tails, GELU, mm."""
    import numpy as np

    path = os.path.join(ROOT, "tests", "golden", "reference_cpu_outputs_next.npz")
    with np.load(path) as data:
        return {k: data[k] for k in data.files}


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    path = os.path.join(ROOT, "tests", "golden", "reference_cpu_outputs.npz")
    return np.load(path)
