"""
pytest configuration: the ``gpu`` marker and shared helpers.

``-m "not gpu"`` runs anywhere (oracle vs. golden vectors, host logic, C-ABI symbol checks);
``-m gpu`` needs a B200 and calls the CUDA kernels through the C ABI.
"""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (B200, sm_100a)')


def pytest_collection_modifyitems(config, items):
    """GPU tests fail loudly, not silently, when selected on a machine without a GPU."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    selected = config.getoption('-m') or ''
    if 'gpu' in selected and 'not gpu' not in selected:
        return  # explicitly requested: let them run and fail
    skip = pytest.mark.skip(reason='needs a CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)
