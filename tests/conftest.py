"""Shared pytest configuration: registers the ``gpu`` marker and skips GPU tests when no CUDA device exists."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the native library")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test, fail if a kernel recorded a bounded-wait failure."""
    yield
    if "gpu" in request.keywords and torch.cuda.is_available():
        from dart_pytorch_b200 import _native
        if _native.available():
            _native.raise_on_device_error()
