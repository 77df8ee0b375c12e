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


@pytest.fixture(scope="session")
def golden_cuda_quant():
    """Outputs of the reference's CUDA quantiser run on the host (tests/golden/make_golden_cuda_quant.py)."""
    import numpy as np
    return np.load(GOLDEN / "cuda_quant_reference.npz")


def cuda_quant_case(g, name):
    """(source tensor view as torch CPU tensor, sr, rht, seed, given scale or None, wanted (data, scale, pts))."""
    import numpy as np
    import torch
    kind, is_bf16, sr, rht, seed, given = (int(v) for v in g[f"{name}_meta"])
    raw = g["base_" + str(g[f"{name}_base"])]
    base = torch.from_numpy(raw.view(np.int16)).view(torch.bfloat16) if is_bf16 else torch.from_numpy(raw)
    x = base if kind == 0 else base.t() if kind == 1 else base[::2, ::2]
    pts = g[f"{name}_pts"]
    return x, bool(sr), bool(rht), seed, (float(pts[0]) if given else None), (g[f"{name}_data"], g[f"{name}_scale"], pts[0])
