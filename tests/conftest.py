import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _native_lib():
    """Build the native library once per session (no-op when it is current)."""
    from cann_hccl_b200 import build
    build.build()
    # small staging buffers and short timeouts keep CPU tests fast and make the staging loop run
    os.environ.setdefault("HCCL_EXEC_TIMEOUT_MS", "20000")
    yield
