import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # GPU tests are skipped (not failed) on machines without a GPU when selected by accident.
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


@pytest.fixture(scope="session")
def ctx():
    import torch
    import cuda_ltc_b200
    c = cuda_ltc_b200.Context(0)
    yield c
    torch.cuda.synchronize()
    assert c.device_status() == 0, "a kernel left a non-zero device status word"
    c.close()
