import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def cuda_device():
    """The B200 the GPU tests run on.  No device -> the GPU tests are skipped; a device without the
    built library -> they fail (there is no fallback to fall back to)."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tritonbench_b200 import lib

    lib.load()
    return torch.device("cuda", 0)
