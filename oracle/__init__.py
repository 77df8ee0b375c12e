"""ctypes front end of the CPU oracle (``liboracle.so``, built from ``nvfp4_oracle.c``,
``adamw_oracle.c`` and ``comfy_oracle.c`` by ``oracle/Makefile``).

TEST INFRASTRUCTURE ONLY.  The oracle restates the reference's NVFP4 arithmetic on the CPU so that
the CUDA kernels can be checked bit for bit; it is also the timed CPU baseline of the benchmark.
Only the test-suite, the smoke test and the benchmark's CPU-baseline leg may import this package.
The product package never does and fails loudly when its CUDA library is missing.

Arrays are numpy; BF16/FP16 tensors travel as ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = None

F32, BF16, F16 = 0, 1, 2
RNE, SR_HASH, SR_PHILOX, SR_MIX = 0, 1, 2, 3


def build(force: bool = False) -> Path:
    """Compile the oracle with the system gcc (a second or two)."""
    target = _HERE / "liboracle.so"
    sources = [_HERE / "nvfp4_oracle.c", _HERE / "adamw_oracle.c", _HERE / "comfy_oracle.c"]
    if force or not target.exists() or any(s.stat().st_mtime > target.stat().st_mtime for s in sources):
        subprocess.run(["make", "-C", str(_HERE), "-B", "liboracle.so"], check=True, capture_output=True)
    return target


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(str(build()))
        L = _LIB
        L.orc_f32_to_bf16.restype = C.c_uint16; L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_f32_to_f16.restype = C.c_uint16; L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_f16_to_f32.restype = C.c_float; L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_e4m3.restype = C.c_uint8; L.orc_f32_to_e4m3.argtypes = [C.c_float]
        L.orc_e4m3_to_f32.restype = C.c_float; L.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_f32_to_e2m1_rne.restype = C.c_uint8; L.orc_f32_to_e2m1_rne.argtypes = [C.c_float]
        L.orc_e2m1_to_f32.restype = C.c_float; L.orc_e2m1_to_f32.argtypes = [C.c_uint8]
        L.orc_cvt_rs_e2m1x4.restype = C.c_uint16; L.orc_cvt_rs_e2m1x4.argtypes = [C.c_float] * 4 + [C.c_uint32]
        L.orc_hash32.restype = C.c_uint32; L.orc_hash32.argtypes = [C.c_uint32, C.c_uint32]
        L.orc_philox4x32_10.restype = None
        L.orc_philox4x32_10.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_scale_offset.restype = C.c_int64; L.orc_scale_offset.argtypes = [C.c_int64] * 3
        L.orc_amax.restype = C.c_float
        L.orc_amax.argtypes = [C.c_void_p, C.c_int] + [C.c_int64] * 4
        L.orc_pts.restype = C.c_float; L.orc_pts.argtypes = [C.c_float, C.c_float, C.c_int]
        L.orc_quantize.restype = None
        L.orc_quantize.argtypes = ([C.c_void_p, C.c_int] + [C.c_int64] * 6 + [C.c_int, C.c_int, C.c_void_p,
                                   C.c_uint32, C.c_float, C.c_int, C.c_void_p, C.c_void_p])
        L.orc_dequantize.restype = None
        L.orc_dequantize.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]
        L.orc_decode_unscaled.restype = None
        L.orc_decode_unscaled.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]
        L.orc_rescale.restype = None
        L.orc_rescale.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_int64, C.c_int64,
                                  C.c_int64, C.c_int, C.c_void_p]
        _bind_comfy(L)
    return _LIB


def _bind_comfy(L):
    L.orc_comfy_bf.restype = C.c_float; L.orc_comfy_bf.argtypes = [C.c_uint16]
    L.orc_comfy_rb.restype = C.c_uint16; L.orc_comfy_rb.argtypes = [C.c_float]
    L.orc_comfy_f8.restype = C.c_float; L.orc_comfy_f8.argtypes = [C.c_uint8]
    L.orc_comfy_rf8.restype = C.c_uint8; L.orc_comfy_rf8.argtypes = [C.c_float]
    L.orc_comfy_f4.restype = C.c_float; L.orc_comfy_f4.argtypes = [C.c_int]
    L.orc_comfy_mix.restype = C.c_uint32; L.orc_comfy_mix.argtypes = [C.c_uint32]
    L.orc_comfy_rf4.restype = C.c_uint8; L.orc_comfy_rf4.argtypes = [C.c_float, C.c_uint32, C.c_int]
    L.orc_comfy_swizzle.restype = C.c_int64; L.orc_comfy_swizzle.argtypes = [C.c_int64] * 3
    L.orc_comfy_finish_scale.restype = C.c_float; L.orc_comfy_finish_scale.argtypes = [C.c_float]
    L.orc_comfy_dequantize.restype = None
    L.orc_comfy_dequantize.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_int64, C.c_int64]
    L.orc_comfy_rotate.restype = C.c_float
    L.orc_comfy_rotate.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]
    L.orc_comfy_quantize.restype = C.c_float
    L.orc_comfy_quantize.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int, C.c_uint32, C.c_void_p, C.c_void_p]
    L.orc_comfy_transpose_requant.restype = C.c_float
    L.orc_comfy_transpose_requant.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p,
                                              C.c_int64, C.c_int64]
    L.orc_comfy_rope.restype = None
    L.orc_comfy_rope.argtypes = [C.c_void_p] * 3 + [C.c_int64] + [C.c_int] * 4


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def round128(n: int) -> int:
    return (n + 127) // 128 * 128


def dtype_code(a: np.ndarray, kind: str | None = None) -> int:
    """numpy float32 -> F32; uint16 -> BF16 unless kind == 'f16'."""
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.uint16:
        return F16 if kind == "f16" else BF16
    if a.dtype == np.float16:
        return F16
    raise TypeError(f"unsupported oracle dtype {a.dtype}")


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even (vectorised)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(h: np.ndarray) -> np.ndarray:
    return (h.astype(np.uint32) << 16).view(np.float32)


def default_signs(seed: int = 1) -> np.ndarray:
    """The 16 +-1 floats of nvfp4_fast_v2.get_signs (nvfp4_fast_v2.py:145-150); seed 1 there."""
    import torch
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randint(0, 2, (16,), generator=gen).float() * 2 - 1).numpy().copy()


def amax(x: np.ndarray, m=None, k=None, s0=None, s1=None, kind=None) -> float:
    """max |bf16(x)| of the logical view; strides are in elements."""
    base = x if x.dtype != np.float16 else x.view(np.uint16)
    if m is None:
        m, k = x.shape
        s0, s1 = (s // x.itemsize for s in x.strides)
    return float(lib().orc_amax(_ptr(base), dtype_code(x, kind), m, k, s0, s1))


def pts(amax_value: float, factor: float = 1.0, variant: int = 0) -> float:
    return float(lib().orc_pts(C.c_float(amax_value), C.c_float(factor), variant))


def quantize(x: np.ndarray, *, sr_mode=RNE, rht=False, signs=None, seed=0, pts_value=None, transpose=False,
             hi_first=False, kind=None, variant=0):
    """Quantise the 2-D array x (or its transpose) to (packed[mp,kp/2], scales[mp/128*32,kp/64*16], pts).

    Mirrors quantize() of nvfp4_fast_v2.py:165-194 over quantize_cuda (csrc/kernels.cu:237-298).
    """
    if x.ndim != 2:
        raise ValueError("oracle quantize expects a 2-D array")
    base = x if x.dtype != np.float16 else x.view(np.uint16)
    m, k = x.shape
    s0, s1 = (s // x.itemsize for s in x.strides)
    if transpose:
        m, k, s0, s1 = k, m, s1, s0
    mp, kp = round128(m), round128(k)
    code = dtype_code(x, kind)
    if pts_value is None:
        a = lib().orc_amax(_ptr(base), code, m, k, s0, s1)
        pts_value = pts(a, 4.0 if rht else 1.0, variant)
    if signs is None:
        signs = default_signs()
    signs = np.ascontiguousarray(signs, dtype=np.float32)
    packed = np.empty((mp, kp // 2), dtype=np.uint8)
    scales = np.empty((mp // 128 * 32, kp // 64 * 16), dtype=np.uint8)
    lib().orc_quantize(_ptr(base), code, m, k, s0, s1, mp, kp, sr_mode, 16 if rht else 0, _ptr(signs),
                       C.c_uint32(seed & 0xFFFFFFFF), C.c_float(pts_value), int(hi_first), _ptr(packed), _ptr(scales))
    return packed, scales, np.float32(pts_value)


def dual(x: np.ndarray, *, sr_mode=RNE, signs=None, seed=0, kind=None):
    """act_pair.dual (act_pair.py:79-102): row packing (no RHT, scale amax/2688, SR seed `seed`) and the
    transposed packing with the sign*H16/4 transform along the rows of x (scale 4*amax/2688, seed+1)."""
    a = amax(x, kind=kind)
    row = quantize(x, sr_mode=sr_mode, rht=False, signs=signs, seed=seed, pts_value=pts(a, 1.0), kind=kind)
    col = quantize(x, sr_mode=sr_mode, rht=True, signs=signs, seed=seed + 1, pts_value=pts(a, 4.0), transpose=True, kind=kind)
    return row, col


def weight_pair(w: np.ndarray, pts_value=None, kind=None):
    """quant_weight_pair / pair() (csrc/kernels.cu:165-185, pair.py:25-49): both contraction
    directions, RNE, no RHT, one shared tensor scale."""
    if pts_value is None:
        pts_value = pts(amax(w, kind=kind), 1.0)
    row = quantize(w, pts_value=pts_value, kind=kind)
    col = quantize(w, pts_value=pts_value, transpose=True, kind=kind)
    return row, col


def dequantize(packed, scales, pts_value, rows, cols, hi_first=False) -> np.ndarray:
    out = np.empty((rows, cols), dtype=np.float32)
    lib().orc_dequantize(_ptr(packed), _ptr(scales), C.c_float(pts_value), packed.shape[1] * 2, rows, cols,
                         int(hi_first), _ptr(out))
    return out


def decode_unscaled(packed, scales, rows=None, cols=None) -> np.ndarray:
    rows = packed.shape[0] if rows is None else rows
    cols = packed.shape[1] * 2 if cols is None else cols
    out = np.empty((rows, cols), dtype=np.float32)
    lib().orc_decode_unscaled(_ptr(packed), _ptr(scales), packed.shape[1] * 2, rows, cols, _ptr(out))
    return out


def rescale(raw: np.ndarray, pts_a, pts_b, rows, cols, *, raw_bf16=True, out_bf16=True, bias=None) -> np.ndarray:
    raw = np.ascontiguousarray(raw, dtype=np.float32)
    out = np.empty((rows, cols), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    lib().orc_rescale(_ptr(raw), int(raw_bf16), C.c_float(pts_a), C.c_float(pts_b), _ptr(b), rows, cols, raw.shape[1],
                      int(out_bf16), _ptr(out))
    return out


def matmul_packed(a, b, rows, cols, *, raw_bf16=True, out_bf16=True, bias=None) -> np.ndarray:
    """scale6.matmul (scale6.py:32-39): block-scaled product in FP32, then the rescale chain.
    a, b are (packed, scales, pts) triples sharing the contraction dimension; result = a @ b.T."""
    import torch
    da = torch.from_numpy(decode_unscaled(a[0], a[1]))
    db = torch.from_numpy(decode_unscaled(b[0], b[1]))
    raw = (da.double() @ db.double().t()).float().numpy()
    return rescale(raw, a[2], b[2], rows, cols, raw_bf16=raw_bf16, out_bf16=out_bf16, bias=bias)


class AdamCfg(C.Structure):
    _fields_ = [("n", C.c_int64), ("master", C.c_int), ("vbits", C.c_int), ("m4", C.c_int), ("nonlinear_m", C.c_int),
                ("block", C.c_int), ("grad_kind", C.c_int), ("grad_cols", C.c_int64), ("grad_stride", C.c_int64),
                ("sa", C.c_float), ("sb", C.c_float), ("add_extra", C.c_int), ("lr", C.c_float), ("decay", C.c_float),
                ("b1", C.c_float), ("b2", C.c_float), ("c1", C.c_float), ("c2", C.c_float), ("eps", C.c_float),
                ("step", C.c_uint32), ("key", C.c_uint32), ("want_amax", C.c_int)]


# storage format -> (master, variance bits, momentum bits)   (engine6.py:13-17)
FORMATS = {"tile32": (32, 16, 8), "fp32_v8": (32, 8, 8), "split24_v16": (24, 16, 8), "split24_v8": (24, 8, 8),
           "sr16_v8": (16, 8, 8), "split24_m4": (24, 8, 4), "sr16_m4": (16, 8, 4), "sr16_m4v4": (16, 4, 4), "half16_v16": (17, 16, 8), "half16_v8": (17, 8, 8), "half16_m8v4": (17, 4, 8),
           "half16_m4v4": (17, 4, 4), "half16_m4v4_sqrt": (17, 4, 4), "float8_v8": (8, 8, 8),
           "float8_m4v4_sqrt": (8, 4, 4), "half16_v8b64": (17, 8, 8), "half16_v8b128": (17, 8, 8), "half16_v8b256": (17, 8, 8)}


def state_block(fmt: str) -> int:
    return int(fmt.split("v8b")[1]) if "v8b" in fmt else 512


def adam_hyper(lr, betas, eps, weight_decay, t):
    """The scalar arguments exactly as engine6.py:88-91 computes them (Python doubles, rounded to FP32 at launch)."""
    import math
    b1, b2 = betas
    return dict(lr=lr, decay=1 - lr * weight_decay, b1=b1, b2=b2, c1=1 / (1 - b1 ** t), c2=1 / math.sqrt(1 - b2 ** t), eps=eps)


def adam_update(fmt, p, grad, m, v, ms, vs, *, step, key, hyper, tail=None, unit=None, grad_kind=0, grad_cols=1,
                grad_stride=1, sa=1.0, sb=1.0, extra=None, want_amax=True, master=None):
    """adam_kernel.update (adam_kernel.py:30-204) in place on numpy arrays; returns per-block amax partials."""
    mst, vb, mb = FORMATS[fmt]
    if master is not None:
        mst = master
    n = p.size
    block = state_block(fmt)
    tiles = (n + block - 1) // block
    part = np.zeros(tiles, dtype=np.float32)
    cfg = AdamCfg(n=n, master=mst, vbits=vb, m4=int(mb == 4), nonlinear_m=int(fmt.endswith("_sqrt")), block=block,
                  grad_kind=grad_kind, grad_cols=grad_cols, grad_stride=grad_stride, sa=sa, sb=sb,
                  add_extra=int(extra is not None), step=step & 0xFFFFFFFF, key=key & 0xFFFFFFFF, want_amax=int(want_amax),
                  **{k: float(val) for k, val in hyper.items()})
    L = lib()
    L.orc_adam_update.restype = None
    L.orc_adam_update.argtypes = [C.c_void_p] * 11
    L.orc_adam_update(C.byref(cfg), _ptr(p), _ptr(grad), _ptr(extra), _ptr(m), _ptr(v), _ptr(ms), _ptr(vs), _ptr(tail),
                      _ptr(unit), _ptr(part))
    return part


def adam_update_plain(p, g, m, v, hyper):
    """optimizer_v5._update with FP32 moments (tensors below 4096 elements); returns amax of the BF16-rounded result."""
    L = lib()
    L.orc_adam_update_plain.restype = None
    L.orc_adam_update_plain.argtypes = [C.c_int64] + [C.c_void_p] * 4 + [C.c_float] * 7 + [C.c_void_p]
    out = np.zeros(1, dtype=np.float32)
    h = hyper
    L.orc_adam_update_plain(p.size, _ptr(p), _ptr(g), _ptr(m), _ptr(v), h["lr"], h["decay"], h["b1"], h["b2"], h["c1"],
                            h["c2"], h["eps"], _ptr(out))
    return float(out[0])


def finish_scale(part: np.ndarray) -> np.float32:
    L = lib()
    L.orc_finish_scale.restype = C.c_float
    L.orc_finish_scale.argtypes = [C.c_void_p, C.c_int64]
    part = np.ascontiguousarray(part, dtype=np.float32)
    return np.float32(L.orc_finish_scale(_ptr(part), part.size))


def split_init(src: np.ndarray, master: int):
    L = lib()
    L.orc_split_init.restype = None
    L.orc_split_init.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p]
    src = np.ascontiguousarray(src, dtype=np.float32)
    hi = np.empty(src.shape, dtype=np.uint16)
    tail = np.empty(src.shape, dtype=np.int8) if master == 24 else None
    L.orc_split_init(_ptr(src), src.size, master, _ptr(hi), _ptr(tail))
    return hi, tail


def e4m3_values() -> np.ndarray:
    """float32 value of each of the 256 E4M3 codes (0x7f / 0xff are NaN)."""
    L = lib()
    return np.array([L.orc_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)


def fp8_decoded(p: np.ndarray, unit: np.ndarray) -> np.ndarray:
    """master8.decoded (master8.py:14-23): BF16 bit patterns of e4m3(p) * unit[flat index // 512], same shape as p."""
    flat = p.reshape(-1)
    scale = np.repeat(np.asarray(unit, dtype=np.float32), 512)[: flat.size]
    with np.errstate(invalid="ignore"):
        return to_bf16_bits(e4m3_values()[flat] * scale).reshape(p.shape)


def fp8_weight_pair(p: np.ndarray, unit: np.ndarray, pts_value: float):
    """master8.encode (master8.py:36-56): both contraction directions of the decoded weight, RNE, one tensor scale."""
    return weight_pair(fp8_decoded(p, unit), pts_value=pts_value)


def philox(ctr, key):
    c = np.asarray(ctr, dtype=np.uint32); k = np.asarray(key, dtype=np.uint32); o = np.empty(4, dtype=np.uint32)
    lib().orc_philox4x32_10(_ptr(c), _ptr(k), _ptr(o))
    return o


# ---- packed-checkpoint (Comfy order) LoRA backend --------------------------------------------------------------------
def comfy_signs(seed: int = 0) -> np.ndarray:
    """128 random +-1 floats of a PackedNVFP4Linear (src/precision_lora/packed.py:104-105)."""
    import torch
    gen = torch.Generator().manual_seed(int(seed) % (2 ** 63))
    return (torch.randint(0, 2, (128,), generator=gen) * 2 - 1).float().numpy()


def comfy_quantize(x_bits: np.ndarray, signs=None, *, sr=False, seed=0):
    """x_bits: uint16 BF16 patterns [rows, cols], cols % 128 == 0 -> (q [rows16, cols/2], s flat swizzled, g)."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    rows, cols = x_bits.shape
    assert cols % 128 == 0
    rows16, rows128 = (rows + 15) // 16 * 16, round128(rows)
    q = np.zeros((rows16, cols // 2), dtype=np.uint8)
    s = np.zeros(rows128 * cols // 16, dtype=np.uint8)
    sg = None if signs is None else np.ascontiguousarray(signs, dtype=np.float32)
    g = lib().orc_comfy_quantize(_ptr(x_bits), rows, cols, _ptr(sg), int(sr), int(seed) & 0xFFFFFFFF, _ptr(q), _ptr(s))
    return q, s, np.float32(g)


def comfy_dequantize(q: np.ndarray, s: np.ndarray, g) -> np.ndarray:
    """-> uint16 BF16 patterns [n, k]."""
    q = np.ascontiguousarray(q, dtype=np.uint8)
    n, k = q.shape[0], q.shape[1] * 2
    y = np.zeros((n, k), dtype=np.uint16)
    lib().orc_comfy_dequantize(_ptr(q), _ptr(np.ascontiguousarray(s, dtype=np.uint8)), float(g), _ptr(y), n, k)
    return y


def comfy_backward_scale(q, s, g, signs) -> np.float32:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    n, k = q.shape[0], q.shape[1] * 2
    amax = lib().orc_comfy_transpose_requant(_ptr(q), _ptr(np.ascontiguousarray(s, dtype=np.uint8)), float(g),
                                             _ptr(np.ascontiguousarray(signs, dtype=np.float32)), 0.0, None, None, n, k)
    return np.float32(lib().orc_comfy_finish_scale(amax))


def comfy_transpose_requant(q, s, g, signs, backward_scale):
    q = np.ascontiguousarray(q, dtype=np.uint8)
    n, k = q.shape[0], q.shape[1] * 2
    qt = np.zeros((k, n // 2), dtype=np.uint8)
    st = np.zeros(k * n // 16, dtype=np.uint8)
    lib().orc_comfy_transpose_requant(_ptr(q), _ptr(np.ascontiguousarray(s, dtype=np.uint8)), float(g),
                                      _ptr(np.ascontiguousarray(signs, dtype=np.float32)), float(backward_scale), _ptr(qt),
                                      _ptr(st), n, k)
    return qt, st


def comfy_rope(x_bits, rot_bits, pairs, backward=False):
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    _, rows, heads, dim = x_bits.shape
    y = np.zeros_like(x_bits)
    lib().orc_comfy_rope(_ptr(x_bits), _ptr(np.ascontiguousarray(rot_bits, dtype=np.uint16)), _ptr(y), rows, heads, dim,
                         int(pairs), int(backward))
    return y


def comfy_matmul(a, b, rows, cols) -> np.ndarray:
    """BF16 result (as float32 values) of the block-scaled product of two Comfy-order packings (q, s, g):
    float64 accumulation of code * block scale, times g_a * g_b in FP32, one rounding to BF16."""
    (qa, sa, ga), (qb, sb, gb) = a, b
    da = from_bf16_bits(comfy_dequantize(qa, sa, 1.0)).astype(np.float64)   # scale 1: e2m1 * e4m3 is exact in BF16
    db = from_bf16_bits(comfy_dequantize(qb, sb, 1.0)).astype(np.float64)
    acc = (da[:rows] @ db[:cols].T).astype(np.float32)
    return from_bf16_bits(to_bf16_bits(acc * (np.float32(ga) * np.float32(gb))))
