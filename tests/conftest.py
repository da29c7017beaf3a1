"""Shared pytest setup: marker registration and import paths.

The package directory `flashattention-cuda_b200/` is not an importable name, so (like the reference's
own conftest, tests/conftest.py:15-17, which puts its repo root on sys.path) it is added to
sys.path here; `import fa_kernels` then resolves to the B200 implementation of that API.
"""

from __future__ import annotations

import os
import sys

import pytest

REPO_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(REPO_ROOT, "flashattention-cuda_b200")
GOLDEN_DIR = os.path.join(REPO_ROOT, "tests", "golden")
for p in (PKG_DIR, REPO_ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_cuda = torch.cuda.is_available()
    except Exception:
        has_cuda = False
    if has_cuda:
        return
    skip = pytest.mark.skip(reason="needs a CUDA GPU")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    def load(name):
        return np.load(os.path.join(GOLDEN_DIR, name))
    return load


@pytest.fixture(autouse=True)
def _device_status_is_clean(request):
    """After every GPU test: no kernel of the test left an error in a device status word (a masked
    block-table entry, a pipeline wait that gave up).  Tests that provoke a flag clear it themselves."""
    yield
    if "gpu" not in request.keywords:
        return
    import torch
    if not torch.cuda.is_available():
        return
    from fa_kernels import _status
    if _status._buffers:
        assert _status.read_status() == 0, "a kernel of this test recorded a device status: " + hex(_status.read_status())
