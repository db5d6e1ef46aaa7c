"""pytest configuration: import paths, the ``gpu`` marker and one-time native builds."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "torch-projectors_b200", ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _native_builds():
    """Build the C oracle (gcc) and the CUDA library (nvcc cross-compiles without a GPU)
    when they are missing or stale."""
    from oracle import build_oracle
    build_oracle.build()
    from torch_projectors_b200 import build as cuda_build
    try:
        cuda_build.build()
    except Exception:
        # a machine without nvcc keeps whatever prebuilt library travelled with the tree
        if not cuda_build.LIB_PATH.exists():
            raise
    yield


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
