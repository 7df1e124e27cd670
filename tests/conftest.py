import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def cpu_kernels(monkeypatch):
    """Puts the plain torch statement of every kernel (tests/kernel_refs.py) in the
    place of the CUDA launchers, so that the code around the kernels runs on the
    CPU.  Test-only: the package has no CPU path of its own."""
    import arle_b200.ops as ops
    import kernel_refs

    for name in kernel_refs.ALL:
        monkeypatch.setattr(ops, name, getattr(kernel_refs, name))
    return ops
