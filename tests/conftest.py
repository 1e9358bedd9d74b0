import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built_libs():
    """Both shared libraries, built on demand (nvcc cross-compiles without a GPU)."""
    from distserve_b200 import build

    return build.build_all()


@pytest.fixture(scope="session")
def golden_dir():
    return ROOT / "tests" / "golden"


@pytest.fixture(autouse=True)
def _first_device_is_current():
    """GPU tests assume cuda:0 is the current device unless they say otherwise."""
    import torch

    if torch.cuda.is_available():
        torch.cuda.set_device(0)
    yield
