import os
import sys

import pytest

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for _p in (os.path.join(_ROOT, "flash-model-architectures_b200"), _ROOT, os.path.dirname(os.path.abspath(__file__))):
    if _p not in sys.path:
        sys.path.insert(0, _p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session", autouse=True)
def _native_library_is_built():
    """The shared library is built once per session (nvcc cross-compiles without a GPU)."""
    sys.path.insert(0, os.path.join(_ROOT, "flash-model-architectures_b200"))
    import build as xma_build

    xma_build.build()


@pytest.fixture()
def device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
