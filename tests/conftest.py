"""Pytest configuration: the ``gpu`` marker, and CPU-only collection hygiene."""

import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
os.environ.setdefault("JIGSAW_LOG_LEVEL", "WARNING")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "multigpu(n): needs n CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch

    have = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for item in items:
        if "gpu" in item.keywords and have == 0:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        m = item.get_closest_marker("multigpu")
        if m is not None and have < int(m.args[0]):
            item.add_marker(pytest.mark.skip(reason=f"needs {m.args[0]} CUDA devices"))
