import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _clean_kernel_status(request):
    """GPU tests start from a clear device status word, so one failure does not cascade."""
    if "gpu" in request.keywords:
        import torch

        if torch.cuda.is_available():
            from agentgarten_b200.ops import native

            if native.available():
                torch.cuda.synchronize()
                native.ext().status(torch.cuda.current_device()).zero_()
    yield
