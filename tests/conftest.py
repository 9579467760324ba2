import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_sessionstart(session):
    """The CUDA library is built in-tree and kept out of history: build it if it is not there yet
    (nvcc cross-compiles without a GPU).  A failed build is left for the tests to report."""
    try:
        from tensor_b200 import build as native_build

        native_build.build()
    except Exception as exc:  # pragma: no cover
        print(f"[conftest] building the CUDA library failed: {exc}")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
