"""FP8-master golden vectors: the reference's Triton kernels on Triton's CPU interpreter (see make_golden.py).

  * `master8.encode` (src/nvfp4_training/_backend/master8.py:36-56): E4M3 weight x per-512 unit -> both NVFP4 orientations,
    and `master8.decoded` (:19-23), on a ragged 65 x 67 weight whose units differ per block;
  * `adam_kernel.update` (adam_kernel.py:108-126) on the update of the reference's own range test
    (tests/test_fp8_master_range.py:36-46): lr 0.25, betas (0, 0), two gradient entries of +-1 in the first and the last
    512-block of a weight stored near 1e-4, so the new value exceeds 448 x unit there and exactly those two units grow.
"""
import math

import numpy as np
import torch


def _u8(t):
    return t.contiguous().view(torch.uint8).numpy().copy()


def make_fp8(out):
    import triton
    from nvfp4_training._backend.adam_kernel import update
    from nvfp4_training._backend.master8 import decoded, encode, unit_for

    blob = {}
    rows, cols = 65, 67
    n = rows * cols
    g = torch.Generator().manual_seed(808)
    w0 = torch.full((rows, cols), 1e-4) * (1 + 0.5 * torch.rand((rows, cols), generator=g))
    u0 = unit_for(w0)
    blocks = triton.cdiv(n, 512)
    unit = torch.full((blocks,), u0, dtype=torch.float32)
    p = (w0 / u0).to(torch.float8_e4m3fn)
    blob["w0"], blob["p0"], blob["unit0"] = w0.numpy().copy(), _u8(p), unit.numpy().copy()
    fmt_master, vb, m4 = 8, 4, True
    m = torch.zeros(n, dtype=torch.uint8)
    ms = torch.zeros(triton.cdiv(n, 64), dtype=torch.float32)
    vs = torch.zeros(triton.cdiv(n, 64), dtype=torch.float32)
    lr, betas, eps, wd = 0.25, (0.0, 0.0), 1e-8, 0.0
    key = 12345
    grads = []
    for step in range(2):
        t = step + 1
        grad = torch.zeros(n)
        grad[1], grad[-1] = 1.0, -1.0
        if step == 1:
            grad = torch.randn(n, generator=g) * 1e-3   # an ordinary step on the grown units
        grads.append(grad.numpy().copy())
        partial = torch.zeros(blocks, dtype=torch.float32)
        b1, b2 = betas
        flat = p.view(-1)
        update[(triton.cdiv(blocks, 2),)](
            flat, grad, m, m, ms, vs, flat, partial, flat, flat, flat, flat, flat, flat, flat, flat, flat, flat,
            unit, flat, flat, n, blocks,
            lr, 1 - lr * wd, b1, b2, 1 / (1 - b1 ** t), 1 / math.sqrt(1 - b2 ** t), eps, t, key,
            False, False, True, False, 1, 1, fmt_master, vb, m4, True, False, 1, 1,
            2, 512, 0, num_warps=4, enable_fp_fusion=False)
        blob[f"s{t}_p"], blob[f"s{t}_unit"] = _u8(p), unit.numpy().copy()
        blob[f"s{t}_m"], blob[f"s{t}_ms"], blob[f"s{t}_vs"] = m.numpy().copy(), ms.numpy().copy(), vs.numpy().copy()
        blob[f"s{t}_part"] = partial.numpy().copy()
    blob["grads"] = np.stack(grads)
    blob["hyper"] = np.array([lr, betas[0], betas[1], eps, wd], dtype=np.float64)
    blob["key"] = np.array([key], dtype=np.int64)
    # both orientations of the grown weight, and of a weight with random per-block units
    p._v6_unit = unit
    plain = decoded(p)
    blob["decoded"] = plain.view(torch.int16).numpy().view(np.uint16).copy()
    scale = plain.float().abs().max() / 2688
    d, s, _, dt, st = encode(p, scale)
    blob.update(enc_scale=scale.numpy().reshape(1).copy(), enc_d=d.numpy().copy(), enc_s=s.numpy().copy(), enc_dt=dt.numpy().copy(),
                enc_st=st.numpy().copy())
    rows2, cols2 = 130, 96
    q = (torch.randn((rows2, cols2), generator=g) * 40).to(torch.float8_e4m3fn)
    units2 = torch.exp2(torch.randint(-12, -6, (triton.cdiv(rows2 * cols2, 512),), generator=g).float())
    q._v6_unit = units2
    plain2 = decoded(q)
    scale2 = plain2.float().abs().max().clamp_min(1e-12) * (1.0 / 2688.0)
    d, s, _, dt, st = encode(q, scale2)
    blob.update(b_p=_u8(q), b_unit=units2.numpy().copy(), b_decoded=plain2.view(torch.int16).numpy().view(np.uint16).copy(),
                b_scale=scale2.numpy().reshape(1).copy(), b_d=d.numpy().copy(), b_s=s.numpy().copy(), b_dt=dt.numpy().copy(),
                b_st=st.numpy().copy())
    np.savez_compressed(out, **blob)
    print("wrote", out, out.stat().st_size, "bytes")
