import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def decode_split():
    """Force the family of decode work splits for one test (``decode_split("unaligned:7")``); cleared afterwards."""

    from dartkv_b200._lib import LIB

    def force(spec):
        LIB.dartkv_decode_split_override(spec.encode() if spec else None)

    yield force
    LIB.dartkv_decode_split_override(None)
