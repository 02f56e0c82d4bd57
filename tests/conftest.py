import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def cuda_lib():
    """Builds (if stale) and loads the CUDA library; GPU tests fail loudly if it is missing."""
    from taraference_b200 import _lib, build
    try:
        build.build()
    except Exception:
        if not build.LIB.exists():
            raise
    return _lib.lib()
