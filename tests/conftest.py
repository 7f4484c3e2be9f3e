import importlib
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) CUDA device")


def _have_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available() and torch.cuda.get_device_capability(0)[0] == 10
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no sm_100 CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def mfk():
    """The product package (its directory name is not a Python identifier)."""
    build = importlib.import_module("test-burn_b200.build")
    try:
        build.build()
    except Exception:
        if not (ROOT / "test-burn_b200" / "libmetallic_cuda.so").exists():
            raise
    return importlib.import_module("test-burn_b200")


@pytest.fixture(scope="session")
def orc():
    import oracle

    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def foundry(mfk):
    import torch

    torch.cuda.set_device(0)
    f = mfk.Foundry(0, torch.cuda.current_stream().cuda_stream)
    yield f
    f.synchronize()
    f.close()
