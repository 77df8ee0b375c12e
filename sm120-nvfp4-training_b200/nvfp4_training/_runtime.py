"""Device gate and lazy loader of the B200 backend (the role of the reference's src/nvfp4_training/_runtime.py:8-18,
with the compute-capability check moved from 12.0 to 10.0 and the JIT build replaced by the prebuilt C-ABI library)."""
from functools import lru_cache


@lru_cache(maxsize=1)
def load_runtime():
    import torch
    if not torch.cuda.is_available() or torch.cuda.get_device_capability()[0] != 10:
        raise RuntimeError("A Blackwell data-center GPU (compute capability 10.x, e.g. B200) is required.")
    from . import _native
    _native.lib()  # raises if the CUDA library is missing: there is no CPU / eager fallback
    from ._backend import engine, quant, step
    from ._backend.linear import AutocastLinear
    return engine, step.StaticStep, quant, AutocastLinear
