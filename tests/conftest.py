import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def native_lib():
    """The built C-ABI library; built here when nvcc is present and the .so is stale."""
    from fleet_chiplet_megakernel_b200 import _build, _cabi
    if _build.needs_build():
        _build.build()
    return _cabi.load()
