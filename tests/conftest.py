"""pytest configuration: the ``gpu`` marker and shared helpers.

``-m "not gpu"`` runs everywhere (oracle vs golden fixtures, host logic, ABI export checks);
``-m gpu`` needs a B200 and calls the CUDA path through the C ABI.
"""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(autouse=True)
def _check_device_status(request):
    """After every GPU test make sure no kernel abandoned a bounded wait."""
    yield
    if "gpu" in request.keywords:
        import torch
        if torch.cuda.is_available():
            from forge_b200 import _lib
            code = _lib.read_status(torch.device("cuda", torch.cuda.current_device()))
            assert code == 0
