import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200 box")


@pytest.fixture(scope="session")
def lib():
    """The CUDA library, built if needed. GPU tests fail (not skip) when it cannot be loaded."""
    from kernl_b200 import _lib, build

    build.build()
    return _lib.load()


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test, make sure no bounded device-side wait expired."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        from kernl_b200 import _lib

        _lib.device_status()

