import os
import sys
from pathlib import Path

import pytest

REPO_ROOT = Path(__file__).resolve().parent.parent
if str(REPO_ROOT) not in sys.path:
    sys.path.insert(0, str(REPO_ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session", autouse=True)
def native_libraries():
    """Builds the native libraries (no-op when up to date) and the CPU checker."""
    from onnx_light_cpu_b200 import build

    build.build_all()
    from oracle import nbits_oracle

    nbits_oracle.build(reference=nbits_oracle.reference_root().is_dir())
    return True


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
