"""Test configuration: the `gpu` marker, the repo root on sys.path, and skip-with-reason
for GPU tests on a machine without a CUDA device."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:  # noqa: BLE001
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device: GPU parity tests run on a B200")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
