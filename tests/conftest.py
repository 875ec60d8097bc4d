import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (sm_100a); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has = torch.cuda.is_available()
    except Exception:                                   # noqa: BLE001
        has = False
    if has:
        return
    skip = pytest.mark.skip(reason="no CUDA GPU here")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(autouse=True)
def _free_device_memory_holds_nan(request):
    """Before every GPU test the allocator's free blocks are filled with NaN, so that a kernel that reads memory nobody
    wrote (a buffer from ``torch.empty``, a row past the step's rows, data its predecessor has not produced yet) turns
    its result into NaN instead of passing on whatever an earlier test left there."""
    if "gpu" in request.keywords:
        import torch
        if torch.cuda.is_available():
            junk = [torch.full((1 << 22,), float("nan"), device="cuda") for _ in range(8)]        # 8 x 16 MB
            junk += [torch.full((n,), float("nan"), device="cuda") for n in (1 << 18, 1 << 14, 1 << 10) for _ in range(8)]
            del junk
    yield
