import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _clear_device_status(request):
    """The tensor-core kernels keep a sticky device status word once a bounded wait runs out;
    reset it so one failing test does not fail the ones after it."""
    if "gpu" in request.keywords:
        import torch
        if torch.cuda.is_available():
            import pkg
            pkg.load().lib().xb_device_status_clear()
    yield
