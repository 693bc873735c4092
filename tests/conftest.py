import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    class G:
        def __getitem__(self, name):
            return np.load(ROOT / "tests" / "golden" / f"{name}.npz", allow_pickle=False)

    return G()


@pytest.fixture(scope="session")
def cuda_lib():
    """The CUDA library, loaded or the test fails: there is no fallback path to fall back to."""
    import torch

    assert torch.cuda.is_available(), "gpu-marked test running without a CUDA device"
    from tenzo_b200 import load_library

    return load_library()
