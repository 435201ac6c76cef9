import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200")


def _ensure_library():
    """The package refuses to import without its shared library; build it if this
    is a fresh checkout (nvcc cross-compiles without a GPU)."""
    import importlib.util
    path = os.path.join(ROOT, "clusterfusionplus_b200", "build.py")
    spec = importlib.util.spec_from_file_location("_cfb200_build", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()


_ensure_library()


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
