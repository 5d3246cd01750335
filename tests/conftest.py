"""Shared pytest configuration.

`gpu` marks the parity tests proper: they call the CUDA kernels through the C
ABI and need a B200.  Everything else (the oracle against the committed golden
vectors, host logic, symbol checks, gloo multi-process tests) runs on CPU.
"""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device: the attention path has no CPU fallback")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
