import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_sessionfinish(session, exitstatus):
    """A run against the range-checking build of the library (AB_BOUNDS_CHECK=1) fails if any kernel recorded an index
    outside its array, whatever the individual tests compared."""
    if os.environ.get("AB_BOUNDS_CHECK") != "1":
        return
    import torch
    if not torch.cuda.is_available():
        return
    from albatross_b200 import _lib
    status = _lib.device_status()
    if status & 16:
        print("\nAB_BOUNDS_CHECK: a kernel recorded an out-of-range index (device status %d)" % status)
        session.exitstatus = 1
