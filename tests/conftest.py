import os
import sys
import warnings

# The compiled reference runs OpenMP regions and OpenBLAS's own thread pool side by side; with
# OpenMP's default active spinning the two oversubscribe a small host (6x slower measured).
# Must be set before anything loads libgomp.
os.environ.setdefault("OMP_WAIT_POLICY", "PASSIVE")

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The compiled reference switches the calling thread to flush-to-zero, which makes numpy
# print a harmless warning about subnormals.
warnings.filterwarnings("ignore", message="The value of the smallest subnormal")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def built_library():
    """Path of libdeepity_b200.so, building it first when nvcc is available."""
    from deepity_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.LIB_PATH
