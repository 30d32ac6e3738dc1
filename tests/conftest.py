import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "slow: long-running test")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _fresh_caches():
    import nabla_b200 as nb

    nb._clear_caches()
    nb.seed(0)
    yield


@pytest.fixture
def mesh_2x4():
    import nabla_b200 as nb

    return nb.DeviceMesh("mesh", (2, 4), ("dp", "tp"))


@pytest.fixture
def mesh_4():
    import nabla_b200 as nb

    return nb.DeviceMesh("mesh1d", (4,), ("x",))
