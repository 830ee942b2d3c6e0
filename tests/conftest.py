import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def native_lib():
    """The C-ABI library, built on demand (nvcc cross-compiles without a GPU)."""
    from cuda_hgemm_b200 import _native, build

    if not _native.LIB_PATH.exists():
        build.build_library()
    return _native.load()


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    major, _ = torch.cuda.get_device_capability(0)
    if major != 10:
        pytest.fail("the GEMM library only runs on sm_100 devices; there is no fallback to test")
    return torch.device("cuda:0")
