import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session", autouse=True)
def _native_built():
    """The product has no CPU fallback: build the native library once for the session."""
    from fastgate_b200 import build

    build.build_all()
    yield
