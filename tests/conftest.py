import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def built_lib():
    """The in-tree shared library, built on demand."""
    from ocannl_b200 import build
    build.build_library()
    return build.LIB


@pytest.fixture(scope="session")
def device(built_lib):
    from ocannl_b200 import backend
    return backend.Device(0)
