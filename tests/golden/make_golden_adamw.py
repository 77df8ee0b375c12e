"""AdamW golden vectors: executes the reference's Triton `update` / `split_init` / `_update` / `_finish_scale`
kernels on Triton's CPU interpreter (see make_golden.py and triton_cpu_shim.py) with the argument list the
reference's engine builds (src/nvfp4_training/_backend/engine6.py:44-104)."""
import math

import numpy as np
import torch


def _bits(t):
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy().copy()
    return t.contiguous().numpy().copy()


FORMATS = {'tile32': (32, 16, 8), 'split24_v8': (24, 8, 8), 'half16_v8': (17, 8, 8), 'half16_v8b128': (17, 8, 8),
           'sr16_v8': (16, 8, 8), 'half16_m4v4_sqrt': (17, 4, 4), 'float8_m4v4_sqrt': (8, 4, 4), 'half16_m8v4': (17, 4, 8),
           'split24_m4': (24, 8, 4), 'sr16_m4': (16, 8, 4), 'sr16_m4v4': (16, 4, 4), 'float8_v8': (8, 8, 8)}
LAUNCH = {'tile32': (2, 4), 'split24_v8': (2, 8), 'half16_v8': (8, 8), 'half16_v8b128': (8, 4), 'sr16_v8': (4, 4),
          'half16_m4v4_sqrt': (1, 4), 'float8_m4v4_sqrt': (2, 4), 'half16_m8v4': (4, 4),
          'split24_m4': (2, 4), 'sr16_m4': (4, 8), 'sr16_m4v4': (1, 4), 'float8_v8': (4, 4)}


def make_adamw(out):
    import triton
    from nvfp4_training._backend.adam_kernel import split_init, update
    from nvfp4_training._backend.optimizer_v5 import _update, _finish_scale
    from nvfp4_training._backend.master8 import unit_for

    blob = {}
    rows, cols, stride = 9, 520, 640          # 4680 elements: ragged last state block
    n = rows * cols
    lr, betas, eps, wd = 3e-4, (0.9, 0.95), 1e-8, 0.1
    g = torch.Generator().manual_seed(2024)
    w0 = torch.randn(n, generator=g) * 0.02
    w0[::97] *= 1e-3                          # FP16-subnormal range for the master SR branch
    w0[5] = 0.0
    raws = [(torch.randn((rows, stride), generator=g) * 40).bfloat16() for _ in range(2)]
    dense = torch.randn(n, generator=g) * 1e-3
    extra = torch.randn(n, generator=g) * 1e-4
    sa, sb = torch.tensor(3.1e-4), torch.tensor(7.7e-2)
    blob.update(w0=w0.numpy(), raw0=_bits(raws[0]), raw1=_bits(raws[1]), dense=dense.numpy(), extra=extra.numpy(),
                scales=np.array([sa.item(), sb.item()], dtype=np.float32),
                meta=np.array([rows, cols, stride], dtype=np.int64),
                hyper=np.array([lr, betas[0], betas[1], eps, wd], dtype=np.float64))
    for fmt, (master, vb, mb) in FORMATS.items():
        width = int(fmt.split('v8b')[1]) if 'v8b' in fmt else 512
        tiles = triton.cdiv(n, width)
        group, warps = LAUNCH[fmt]
        key = 12345 + 7919 * 3
        # master storage
        unit = tail = None
        if master == 32:
            p = w0.clone()
        elif master == 8:
            u0 = unit_for(w0)
            unit = torch.full((triton.cdiv(n, 512),), u0, dtype=torch.float32)
            p = (w0 / u0).to(torch.float8_e4m3fn)
        else:
            p = torch.empty(n, dtype=torch.float16 if master == 17 else torch.bfloat16)
            tail = torch.empty(n, dtype=torch.int8) if master == 24 else p
            split_init[(triton.cdiv(n, 512),)](w0, p, tail, n, master == 24, 512)
            if master != 24:
                tail = None
        blob[f"{fmt}_p0"] = _bits(p)
        if tail is not None:
            blob[f"{fmt}_tail0"] = tail.numpy().copy()
        if unit is not None:
            blob[f"{fmt}_unit0"] = unit.numpy().copy()
        m = torch.zeros((n + 1) // 2 if mb == 4 and vb != 4 else n, dtype=torch.uint8 if mb == 4 else torch.int8)
        ms = torch.zeros(triton.cdiv(n, 64 if mb == 4 else width), dtype=torch.float32)
        vs = torch.zeros(triton.cdiv(n, 64 if vb == 4 else width), dtype=torch.float32)
        v = None
        if vb != 4 or mb != 4:
            v = torch.zeros(triton.cdiv(n, 2) if vb == 4 else n, dtype=torch.uint8 if vb < 16 else torch.float16)
        for step in range(3):
            t = step + 1
            b1, b2 = betas
            packed = step < 2
            grad = raws[step] if packed else dense
            add = step == 1
            partial = torch.zeros(tiles, dtype=torch.float32)
            c, st = (cols, stride) if packed else (1, 1)
            update[(triton.cdiv(tiles, group),)](
                p, grad, m, v if v is not None else m, ms, vs, tail if tail is not None else p, partial,
                sa if packed else p, sb if packed else p, extra if add else p, p, p, p, p, p, p, p,
                unit if unit is not None else p, p, p, n, tiles,
                lr, 1 - lr * wd, b1, b2, 1 / (1 - b1 ** t), 1 / math.sqrt(1 - b2 ** t), eps, t, key,
                packed, add, True, False, c, st, master, vb, mb == 4, fmt.endswith("_sqrt"), False, 1, 1,
                group, width, 0, num_warps=warps, enable_fp_fusion=False)
            scale = torch.empty((), dtype=torch.float32)
            _finish_scale[(1,)](partial, scale, tiles, triton.next_power_of_2(tiles))
            blob[f"{fmt}_s{t}_p"] = _bits(p)
            blob[f"{fmt}_s{t}_m"] = m.numpy().copy()
            if v is not None:
                blob[f"{fmt}_s{t}_v"] = _bits(v)
            blob[f"{fmt}_s{t}_ms"], blob[f"{fmt}_s{t}_vs"] = ms.numpy().copy(), vs.numpy().copy()
            blob[f"{fmt}_s{t}_part"] = partial.numpy().copy()
            blob[f"{fmt}_s{t}_scale"] = scale.numpy().reshape(1).copy()
            if tail is not None:
                blob[f"{fmt}_s{t}_tail"] = tail.numpy().copy()
            if unit is not None:
                blob[f"{fmt}_s{t}_unit"] = unit.numpy().copy()
    # small-tensor base path: FP32 p, m, v (optimizer_v5.py:9-53 with COMPACT=False)
    ns = 1000
    ps = (torch.randn(ns, generator=g) * 0.5).float()
    gs = (torch.randn(ns, generator=g) * 0.01).float()
    mm, vv = torch.zeros(ns), torch.zeros(ns)
    blob["plain_p0"], blob["plain_g"] = ps.numpy().copy(), gs.numpy().copy()
    for t in (1, 2):
        b1, b2 = betas
        part = torch.zeros(triton.cdiv(ns, 512))
        _update[(triton.cdiv(ns, 512),)](ps, gs, mm, vv, ps, ps, part, ps, ps, ps, ps, ns, lr, 1 - lr * wd, b1, b2,
                                         1 / (1 - b1 ** t), 1 / math.sqrt(1 - b2 ** t), eps, False, True, False, False, False,
                                         1, 1, 512, num_warps=4, enable_fp_fusion=False)
        blob[f"plain_s{t}_p"], blob[f"plain_s{t}_m"], blob[f"plain_s{t}_v"] = ps.numpy().copy(), mm.numpy().copy(), vv.numpy().copy()
        blob[f"plain_s{t}_part"] = part.numpy().copy()
    np.savez_compressed(out, **blob)
    print("wrote", out, out.stat().st_size, "bytes")
