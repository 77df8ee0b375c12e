"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import oracle as O


def to_oracle(t: torch.Tensor):
    """torch tensor (any strides) -> (numpy view with the same strides, kind) for the oracle."""
    t = t.detach().cpu()
    if t.dtype == torch.float32:
        base = t.numpy()
        return base, None
    kind = "f16" if t.dtype == torch.float16 else None
    # build a numpy array over the same storage with the same strides
    flat = torch.empty(0, dtype=torch.int16).set_(t.untyped_storage()).numpy().view(np.uint16)
    arr = np.lib.stride_tricks.as_strided(flat[t.storage_offset():], shape=tuple(t.shape),
                                          strides=tuple(s * 2 for s in t.stride()))
    return arr, kind


def signs_dev(device="cuda"):
    return torch.from_numpy(O.default_signs()).to(device)


def alloc_packing(rows_p, cols_p, device="cuda", poison=0xCD):
    packed = torch.full((rows_p, cols_p // 2), poison, dtype=torch.uint8, device=device)
    scales = torch.full((rows_p // 128 * 32, cols_p // 64 * 16), poison, dtype=torch.uint8, device=device)
    return packed, scales


def outlier_tensor(shape, seed, dtype=torch.bfloat16, scale=1.0):
    """N(0,1) with 0.1 % of the entries (seeded positions) scaled x50."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g) * scale
    n = x.numel()
    pos = torch.randperm(n, generator=g)[: max(1, n // 1000)]
    x.view(-1)[pos] *= 50
    return x.to(dtype)
