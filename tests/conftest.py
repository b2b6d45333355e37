import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _have_gpu() -> bool:
    try:
        from loadngo_b200 import compute
        g = compute.Gpu(0)
        g.free()
        return True
    except Exception:
        return False


_GPU = None


def pytest_collection_modifyitems(config, items):
    global _GPU
    gpu_items = [i for i in items if "gpu" in i.keywords]
    if not gpu_items:
        return
    if _GPU is None:
        _GPU = _have_gpu()
    if not _GPU:
        skip = pytest.mark.skip(reason="no CUDA device")
        for item in gpu_items:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def gpu():
    from loadngo_b200 import compute
    g = compute.Gpu(0)
    yield g
    g.free()
