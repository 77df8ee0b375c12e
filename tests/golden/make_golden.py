"""Generate golden vectors by executing the reference's own Triton kernels on the CPU.

Run once in the build container, where the reference sources are mounted read-only:

    python tests/golden/make_golden.py /path/to/reference/src

The reference's device code cannot run without an SM120 GPU, but its Triton kernels are Python
functions that Triton's interpreter (TRITON_INTERPRET=1) evaluates with numpy; triton_cpu_shim.py
closes the two gaps of that interpreter (IEEE round-to-nearest casts, the three inline PTX
instructions).  The outputs are stored next to the inputs in small .npz files; the CPU oracle and
the CUDA kernels are both checked against them byte for byte.  No reference source is copied.
"""
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import triton_cpu_shim  # noqa: F401  (must precede the reference imports)

import numpy as np
import torch


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16 or t.dtype == torch.float16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy().copy()
    return t.contiguous().numpy().copy()


def signs16() -> torch.Tensor:
    gen = torch.Generator(device="cpu").manual_seed(1)
    return torch.randint(0, 2, (16,), generator=gen).float() * 2 - 1


def outliers(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g) * scale
    n = x.numel()
    pos = torch.randperm(n, generator=g)[: max(1, n // 1000)]
    x.view(-1)[pos] *= 50
    return x


def make_quant(out: Path):
    from nvfp4_training._backend import act_pair, pair as pair_mod, remat, scale6
    signs = signs16()
    blob = {"signs": signs.numpy()}
    # dual: row packing + RHT-transposed packing from one tile (act_pair.py:79-102)
    cases = [("a", (40, 70), torch.bfloat16, False, 0), ("b", (40, 70), torch.bfloat16, True, 5),
             ("c", (128, 256), torch.bfloat16, False, 0), ("d", (128, 256), torch.bfloat16, True, 173),
             ("e", (193, 129), torch.float32, True, 4294967295), ("f", (130, 300), torch.float32, False, 0)]
    for tag, shape, dtype, sr, seed in cases:
        x = outliers(shape, 100 + len(tag) + shape[0], 1.0).to(dtype)
        row, col = act_pair.dual(x, signs, sr=sr, offset=seed)
        blob[f"dual_{tag}_x"] = bits(x)
        blob[f"dual_{tag}_meta"] = np.array([int(sr), seed, 1 if dtype == torch.bfloat16 else 0], dtype=np.int64)
        for name, p in (("row", row), ("col", col)):
            blob[f"dual_{tag}_{name}_data"] = p.data.numpy()
            blob[f"dual_{tag}_{name}_scale"] = p.scale.numpy()
            blob[f"dual_{tag}_{name}_pts"] = p.pts.numpy().reshape(1)
    # weight pair (pair.py:38-49) and single orientation (remat.py:21-28)
    for tag, shape, dtype in (("a", (100, 200), torch.float32), ("b", (128, 512), torch.float16), ("c", (257, 130), torch.bfloat16)):
        w = (outliers(shape, 7 + shape[1], 0.02)).to(dtype)
        amax = w.bfloat16().abs().amax().float() if dtype != torch.float16 else w.float().bfloat16().abs().amax().float()
        pts = torch.clamp_min(amax, 1e-12) * (1.0 / 2688.0)
        d, s, _, dt, st = pair_mod.pair(w, pts, (64, 128, 4))
        blob[f"pair_{tag}_w"] = bits(w)
        blob[f"pair_{tag}_kind"] = np.array([{torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[dtype]])
        blob[f"pair_{tag}_pts"] = pts.numpy().reshape(1)
        blob[f"pair_{tag}_data"], blob[f"pair_{tag}_scale"] = d.numpy(), s.numpy()
        blob[f"pair_{tag}_data_t"], blob[f"pair_{tag}_scale_t"] = dt.numpy(), st.numpy()
        for tr in (False, True):
            sd, ss = remat.single(w, pts, tr)
            blob[f"single_{tag}_{int(tr)}_data"], blob[f"single_{tag}_{int(tr)}_scale"] = sd.numpy(), ss.numpy()
    # post-GEMM rescale (scale6.py:7-30)
    g = torch.Generator().manual_seed(11)
    for tag, raw_dtype, out_dtype, with_bias in (("a", torch.bfloat16, torch.bfloat16, True), ("b", torch.bfloat16, torch.float32, False),
                                                 ("c", torch.float32, torch.float32, True), ("d", torch.bfloat16, torch.bfloat16, False)):
        raw = (torch.randn((128, 256), generator=g) * 300).to(raw_dtype)
        sa = torch.tensor(0.00123, dtype=torch.float32)
        sb = torch.tensor(0.0000317, dtype=torch.float32)
        bias = (torch.randn(200, generator=g)).to(torch.bfloat16 if tag == "a" else torch.float32) if with_bias else None
        y = scale6.rescale(raw, sa, sb, 100, 200, out_dtype, bias)
        blob[f"rescale_{tag}_raw"] = bits(raw)
        blob[f"rescale_{tag}_meta"] = np.array([raw_dtype == torch.bfloat16, out_dtype == torch.bfloat16, with_bias], dtype=np.int64)
        blob[f"rescale_{tag}_scales"] = np.array([sa.item(), sb.item()], dtype=np.float32)
        if with_bias:
            blob[f"rescale_{tag}_bias"] = bias.float().numpy()
        blob[f"rescale_{tag}_out"] = y.float().numpy()
    np.savez_compressed(out, **blob)
    print("wrote", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to the reference's src directory> [all|quant|...]")
    ref_src = sys.argv[1]
    sys.path.insert(0, ref_src)
    which = sys.argv[2] if len(sys.argv) > 2 else "all"
    if which in ("all", "quant"):
        make_quant(HERE / "quant_reference.npz")
    if which in ("all", "adamw"):
        from make_golden_adamw import make_adamw
        make_adamw(HERE / "adamw_reference.npz")
    if which in ("all", "fp8"):
        from make_golden_fp8 import make_fp8
        make_fp8(HERE / "fp8_master_reference.npz")
