import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "sm120-nvfp4-training_b200"
for p in (str(ROOT), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_quant():
    import numpy as np
    return np.load(GOLDEN / "quant_reference.npz")


@pytest.fixture(scope="session")
def native():
    """The CUDA library through its C ABI; the GPU tests fail loudly if it is missing."""
    import torch
    assert torch.cuda.is_available(), "GPU test selected without a CUDA device"
    from nvfp4_training import _native
    _native.lib()
    return _native
