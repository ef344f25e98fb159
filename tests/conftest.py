import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def lib_path():
    """Builds the operator library if it is missing (nvcc cross-compiles without a GPU)."""
    from tinyflow_b200.build import LIB_PATH, build
    if not os.path.exists(LIB_PATH):
        build()
    return LIB_PATH
