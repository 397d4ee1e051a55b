import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device")


def pytest_collection_modifyitems(config, items):
    """Without a device a test marked gpu is reported as skipped, never as passed."""
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device (run with -m 'not gpu' here)")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
