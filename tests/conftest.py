import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")
    config.addinivalue_line("markers", "expects_status: the test provokes a kernel status word on purpose")


@pytest.fixture(scope="session", autouse=True)
def _libraries_present():
    """A fresh checkout has no binaries (they are not versioned): build them once before the first test. An existing
    build is used as it is."""
    from asymgemm_b200 import _lib, build
    if not (_lib.LIB_PATH.exists() and _lib.TORCH_OPS_PATH.exists()):
        build.build()
    yield


@pytest.fixture(autouse=True)
def _status_clean(request):
    """After every GPU test, fail if a kernel left a non-zero status word behind."""
    yield
    if request.node.get_closest_marker("gpu") is not None and not request.node.get_closest_marker("expects_status"):
        import torch
        if torch.cuda.is_available():
            import asymgemm_b200 as ag
            ag.check_status()
