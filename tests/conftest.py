import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU machine)")


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    # A GPU test on a machine without a GPU is an error of invocation, not a pass:
    # skip loudly so that "-m gpu" here never looks green by falling back to anything.
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device: GPU parity tests only run on the GPU machine")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def ctx():
    import primitiv_b200 as pb
    c = pb.Context(0)
    yield c
    c.close()
