import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "multigpu: needs more than one CUDA device")
    config.addinivalue_line("markers", "expect_status: the test provokes a device status word on purpose")


@pytest.fixture(autouse=True)
def _clear_device_status(request):
    """GPU tests start from a clean status block and fail if a kernel recorded a time-out."""
    if request.node.get_closest_marker("gpu") is None:
        yield
        return
    import torch

    from parallelkernelbench_b200 import _native as nv

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    nv.clear_status()
    yield
    if request.node.get_closest_marker("expect_status") is None:
        nv.raise_on_status(sync=True)
