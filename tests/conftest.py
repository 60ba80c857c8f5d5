"""pytest configuration: the ``gpu`` marker and import paths.

``-m "not gpu"`` covers the oracle against the golden vectors, the host-side logic and the
symbol table of the C-ABI library; ``-m gpu`` holds the parity tests proper, which call the
CUDA kernels through the C ABI.
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for sub in ("aihwkit-lightning_b200", "oracle", os.path.join("tests", "golden"), "tests"):
    path = os.path.join(ROOT, sub)
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
