"""Shared pytest configuration: the `gpu` marker and helpers used by both CPU and GPU tests."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_cuda = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_cuda = False
    if has_cuda:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _check_device_status_at_end():
    """After all GPU tests: no kernel may have recorded a timed-out wait."""
    yield
    try:
        import torch

        if torch.cuda.is_available():
            from aitemplate_b200 import kernels

            assert kernels.device_status() == 0, "a kernel recorded a bounded-wait timeout"
    except ImportError:  # pragma: no cover
        pass
