import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multi_gpu: needs more than one CUDA device")
    config.addinivalue_line("markers", "slow: long-running test")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multi_gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _clear_kernel_error_word(request):
    """A GPU test that fails after a bounded device wait gave up must not leave the error word set for the tests
    that follow it in the same process."""
    yield
    if "gpu" in request.keywords or "multi_gpu" in request.keywords:
        try:
            import torch

            if torch.cuda.is_available():
                from areal_b200.ops import lib as oplib

                oplib.kernel_error()
        except Exception:
            pass
