import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import torch

    return torch.load(ROOT / "tests/golden/paged_decode_golden.pt", weights_only=False)


@pytest.fixture(scope="session")
def built_libs():
    """Both shared libraries, built in-tree if stale (cross-compiles without a GPU)."""
    from single_gpu_inference_lab_b200 import build

    return build.build_all()
