"""Test configuration: registers the ``gpu`` marker and the shared helpers.

``-m "not gpu"`` runs the oracle / host-logic / C-ABI-symbol tests on any
machine; ``-m gpu`` runs the parity tests proper on a B200.
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
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The shared library must exist for every test session (built in-tree)."""
    from oasr_b200 import _lib, build

    if not _lib.LIB_PATH.exists():
        build.build()
    return _lib.load()


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After each GPU test no kernel may have abandoned a bounded wait."""
    yield
    if "gpu" in request.keywords:
        import torch

        if torch.cuda.is_available():
            import oasr_b200

            assert oasr_b200.device_status() == 0
