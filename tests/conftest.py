import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 and the built CUDA library")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def lib():
    """The C-ABI library (built on demand; nvcc cross-compiles without a GPU)."""
    from tessera_b200 import _lib, build
    if not _lib.lib_path().exists():
        build.build()
    return _lib.load()
