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
