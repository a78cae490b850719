import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

GOLDEN = os.path.join(REPO, "tests", "golden")


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
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return {name: np.load(os.path.join(GOLDEN, f"{name}.npz")) for name in ("kat", "writer", "config0")}


@pytest.fixture(autouse=True)
def _decode_kernels_report_no_failure(request):
    """After every GPU test: the decode kernels record a bounded wait that gave up, or an
    unexpected shared-memory layout, in a device-side status word instead of hanging or
    faulting; a test must never leave it set."""
    yield
    if "gpu" not in request.keywords:
        return
    import ctypes

    import torch

    if not torch.cuda.is_available():
        return
    from beyond_kv_cache_b200 import _lib

    status = ctypes.c_int(-1)
    _lib.call("bkv_decode_device_status", ctypes.byref(status))
    assert status.value == 0, f"decode kernel status word = {status.value}"
