"""Shared pytest configuration.

Tests that need a CUDA device carry ``@pytest.mark.gpu``; everything else runs
on CPU (multi-process cases over the ``gloo`` backend on 127.0.0.1).
"""

import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# fp32-only test models would otherwise trip the "master_weight_bits has no effect" guard
os.environ.setdefault("FLASHOPTIM_ALLOW_INEFFECTIVE_MASTER_WEIGHT_BITS", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")
    config.addinivalue_line("markers", "thirdparty: tiny random-init third-party models (no network; CPU, ten of them also on the GPU)")


def pytest_collection_modifyitems(config, items):
    import torch

    n_gpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and n_gpu == 0:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and n_gpu < 2:
            item.add_marker(skip_multi)
