import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    # A fresh checkout has no built libraries (they are not tracked): build them once.
    built = [os.path.join(ROOT, "gograd_b200", "liboptengine.so"), os.path.join(ROOT, "gograd_b200", "libgograd_host.so"),
             os.path.join(ROOT, "oracle", "liboptim_oracle.so")]
    if not all(os.path.exists(p) for p in built):
        import __graft_entry__
        __graft_entry__.build()


def pytest_collection_modifyitems(config, items):
    """GPU tests skip themselves on a box without a device instead of failing."""
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
