import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _has_cuda() -> bool:
    # same idea as the reference's skip predicates (python/avelang/testing.py:1-26)
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_cuda():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def built_lib():
    """In-tree shared library, built on demand (nvcc cross-compiles without a GPU)."""
    from avelang_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def checker():
    """The CPU checker modules (test infrastructure)."""
    from oracle import c_oracle, gdn_oracle
    c_oracle.build()
    return gdn_oracle, c_oracle
