"""Test configuration: the ``gpu`` marker and shared helpers.

``-m "not gpu"`` runs everywhere (oracle vs golden vectors, host logic, ABI surface);
``-m gpu`` needs a B200 and calls the kernels through the C ABI.
"""

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


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
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """Build the shared library once per session (a no-op when it is up to date)."""
    from iron_b200.build import build

    build()
