import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _have_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def dev():
    from qubivex_b200.device import CudaDevice
    d = CudaDevice(0, timing=True)
    yield d
    d.close()


@pytest.fixture(scope="session")
def dev_x():
    """A device of the experiment build of the library: the chunk and run-length rules follow the environment."""
    from qubivex_b200.device import CudaDevice
    d = CudaDevice(0, timing=True, experiments=True)
    yield d
    d.close()
