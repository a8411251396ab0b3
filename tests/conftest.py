"""pytest configuration: registers the ``gpu`` marker and skips GPU tests when no
CUDA device is visible (they are selected explicitly with ``-m gpu`` on a B200)."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True, scope="session")
def _poisoned_buffers():
    """Buffers allocated by the ctypes wrappers start as NaN bytes during the tests, so that a read
    of a slot no kernel wrote fails a parity check instead of depending on allocator history."""
    from mhc.cu_b200 import capi
    capi.POISON = True
    yield
    capi.POISON = False
