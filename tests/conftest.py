import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(params=[False, True], ids=["plain", "pdl"])
def pdl(request):
    """Runs the test twice: with ordinary launches and with programmatic dependent launch (every kernel may start
    while the one before it drains, and waits on the device before it reads) - the mode the benchmark times."""

    from tensorfold_b200 import _lib

    was = _lib.set_pdl(request.param)
    yield request.param
    _lib.set_pdl(was)
