import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def lib():
    """The loaded C-ABI library; a GPU test that gets here without it fails loudly."""
    from tcfp_b200 import _C

    return _C.load()


@pytest.fixture(autouse=True)
def _device_status_guard(request):
    """After every GPU test: no kernel may have given up a bounded wait."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import torch

        if torch.cuda.is_available():
            from tcfp_b200 import _C

            _C.check_device_status()
