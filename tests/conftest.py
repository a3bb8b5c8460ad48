import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_sessionstart(session):
    """Builds the native pieces when they are missing or stale (nvcc cross-compiles without
    a GPU), so the suite can run from a fresh checkout."""
    from drivingsdk_b200 import build as native_build
    native_build.build_all(force=False)
    from oracle import msda_oracle
    msda_oracle.build()


def pytest_collection_modifyitems(config, items):
    """GPU tests never run where there is no GPU, whatever -m says."""
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
