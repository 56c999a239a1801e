import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def device_status():
    """Checks after the test that no kernel reported a timed-out wait."""
    yield
    if torch.cuda.is_available():
        from fastfold_b200.ops import _lib
        st = _lib.read_status()
        assert st[0] == 0, "device status word: %s" % st[:5]


@pytest.fixture(autouse=True)
def _poison_free_gpu_memory(request):
    """GPU tests only: fills a block of device memory with 0xFF bytes (NaN as bf16 / fp16 / fp32) and hands it back to the
    caching allocator, so that the ``torch.empty`` workspaces and outputs of the test start out as NaN - a kernel that
    leaves part of its output unwritten, or reads scratch it never filled, then fails its comparison instead of passing
    on stale data of an earlier test."""
    if "gpu" in request.keywords and torch.cuda.is_available():
        free, _ = torch.cuda.mem_get_info()
        n = int(min(2 << 30, free // 4))
        if n > 0:
            blocks = [torch.empty(n // 4, dtype=torch.uint8, device="cuda").fill_(0xFF) for _ in range(4)]
            torch.cuda.synchronize()
            del blocks
    yield
