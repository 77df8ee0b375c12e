"""ctypes binding of libnvfp4_b200.so (the C ABI declared in include/nvfp4_b200.h).

PyTorch supplies device memory and streams only; every kernel on the NVFP4 path lives in the shared
library.  There is no CPU or eager fallback: a missing library raises at first use.
"""
from __future__ import annotations

import ctypes as C
import os
import re
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libnvfp4_b200.so"
_HEADER = Path(__file__).resolve().parents[2] / "include" / "nvfp4_b200.h"
_lib = None

F32, BF16, F16, E4M3 = 0, 1, 2, 3
Q_RHT, Q_SR_HASH, Q_SR_PHILOX, Q_HI_FIRST = 1, 2, 4, 8
_CODES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
_ERRORS = {1: ValueError, 2: ValueError, 3: TypeError, 4: RuntimeError, 5: RuntimeError, 6: NotImplementedError}

P, I64, I32, U32, F = C.c_void_p, C.c_int64, C.c_int, C.c_uint32, C.c_float

_SIGNATURES = {
    "nvfp4_last_error": (C.c_char_p, []),
    "nvfp4_version": (I32, []),
    "nvfp4_amax_scratch_bytes": (I64, []),
    "nvfp4_amax": (I32, [P, I32, I64, I64, I64, I64, P, P, P]),
    "nvfp4_quantize_tile": (I32, [P, I32, I64, I64, I64, I64, P, P, P, P, P, I32, U32, P, P, P, I32, U32, P, P]),
    "nvfp4_quantize_tile_amax": (I32, [P, I32, I64, I64, I64, I64, P, P, P, P, P, P, I32, U32, P, P, P, I32, U32, P, P]),
    "nvfp4_quantize_fp8_weight": (I32, [P, P, I64, I64, P, P, P, P, P, P]),
    "nvfp4_quantize": (I32, [P, I32, I64, I64, I64, I64, I64, I64, I32, I32, U32, P, P, P, I32, P, P, P, P, P, P, P, P]),
    "nvfp4_quantize_static_max_elements": (I64, []),
    "nvfp4_quantize_static": (I32, [P, I32, I64, I64, I64, I64, I64, I64, I32, I32, U32, P, P, P, P, P, P]),
    "nvfp4_dequantize": (I32, [P, P, P, I64, I64, I64, I32, I32, P, I64, P]),
    "nvfp4_adamw_step": (I32, [P, I32, P, I32, I64, I64, P, P, P, F, P, P, P, P, P, P, I64, I32, I32, I32, I32,
                                 F, F, F, F, F, F, F, U32, U32, P, P, P, P]),
    "nvfp4_adamw_step_prepack": (I32, [P, I32, P, I32, I64, I64, P, P, P, F, P, P, P, P, P, I64, I64, I32, I32, I32, I32,
                                         F, F, F, F, F, F, F, U32, U32, P, P, P, P, P, P, P, P, P]),
    "nvfp4_adamw_plain": (I32, [P, P, P, P, I64, F, F, F, F, F, F, F, F, P, P]),
    "nvfp4_split_init": (I32, [P, I64, I32, P, P, P]),
    "nvfp4_rope": (I32, [P, P, P, P, I64, I32, I32, I32, I64, I64, I32, P, P]),
    "nvfp4_rope_qkv_bwd": (I32, [P, I64, P, I64, P, I64, P, P, P, I64, I32, I32, I32, P, P]),
    "nvfp4_swiglu": (I32, [P, I64, P, I64, P, I64, P, I64, P, I64, I64, I64, P, P]),
    "nvfp4_add_rmsnorm": (I32, [P, P, P, F, I64, I64, P, P, P, P, P]),
    "nvfp4_rmsnorm_bwd_partials": (I64, [I64, I64]),
    "nvfp4_rmsnorm_bwd": (I32, [P, P, P, P, P, I64, I64, P, P, P, P, P]),
    "nvfp4_cross_entropy_fwd": (I32, [P, I64, P, I64, I64, P, P, P, P]),
    "nvfp4_cross_entropy_bwd": (I32, [P, I64, P, P, P, I64, I64, P, I64, P, P]),
    "nvfp4_gemm": (I32, [P, P, P, P, P, P, I64, I64, I64, P, I32, P, I32, I64, I64, I64, I32, P, P]),
    "nvfp4_comfy_quantize": (I32, [P, I64, I64, P, I32, U32, P, P, P, P, P, P]),
    "nvfp4_comfy_dequantize": (I32, [P, P, P, P, I64, I64, P]),
    "nvfp4_comfy_backward_scale": (I32, [P, P, P, P, I64, I64, P, P, P]),
    "nvfp4_comfy_transpose_requant": (I32, [P, P, P, P, P, P, P, I64, I64, P]),
    "nvfp4_comfy_finish_scale": (I32, [P, P, P]),
    "nvfp4_comfy_rope": (I32, [P, P, P, I64, I32, I32, I32, I32, P]),
}


def declared_symbols() -> list[str]:
    """Names of the entry points the public header declares."""
    text = _HEADER.read_text()
    return sorted(set(re.findall(r"\b(nvfp4_[a-z0-9_]+)\s*\(", text)))


def lib():
    """Load the CUDA library once; never falls back to another implementation."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(f"{_LIB_PATH} is missing: build it with `python sm120-nvfp4-training_b200/build.py` "
                               "(no CPU or eager fallback exists for the NVFP4 path)")
        handle = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


CALLS = 0   # kernel-launching library calls made by this process (each launches one or two kernels)


def check(code: int) -> None:
    global CALLS
    CALLS += 1
    if code:
        message = lib().nvfp4_last_error().decode("utf-8", "replace")
        raise _ERRORS.get(code, RuntimeError)(message)


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise TypeError(f"Unsupported dtype {t.dtype}; use BF16 autocast / FP32 or FP16 masters") from None


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


_SCRATCH: dict[tuple, torch.Tensor] = {}


def scratch(device: torch.device) -> torch.Tensor:
    """Zero-initialised amax scratch, one per (device, stream): the kernels leave it zeroed again."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _SCRATCH.get(key)
    if buf is None:
        buf = torch.zeros(int(lib().nvfp4_amax_scratch_bytes()), dtype=torch.uint8, device=device)
        _SCRATCH[key] = buf
    return buf


def round128(n: int) -> int:
    if n <= 0:
        raise ValueError("Empty dimensions are not supported")
    return (n + 127) // 128 * 128


def amax(x: torch.Tensor) -> torch.Tensor:
    """float32[4] on the device: amax, scale, 4x scale, true-division scale (see nvfp4_amax)."""
    out = torch.empty(4, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().nvfp4_amax(x.data_ptr(), dtype_code(x), x.shape[0], x.shape[1], x.stride(0), x.stride(1),
                               scratch(x.device).data_ptr(), out.data_ptr(), stream_of(x)))
    return out


def quantize_tile(x, signs, *, row=None, col=None, seed_base=None, amax=None):
    """row / col: None or dict(packed, scales, pts, flags, seed).  amax: device float left by the producer of x; the
    kernel then computes the tensor scales itself and writes them into the pts tensors."""
    def unpack(o):
        if o is None:
            return None, None, None, 0, 0
        return o["packed"].data_ptr(), o["scales"].data_ptr(), o["pts"].data_ptr(), int(o.get("flags", 0)), int(o.get("seed", 0)) & 0xFFFFFFFF
    rp, rs, rq, rf, rsd = unpack(row)
    cp, cs, cq, cf, csd = unpack(col)
    with torch.cuda.device(x.device):
        if amax is not None:
            check(lib().nvfp4_quantize_tile_amax(x.data_ptr(), dtype_code(x), x.shape[0], x.shape[1], x.stride(0), x.stride(1),
                                                 signs.data_ptr(), ptr(seed_base), amax.data_ptr(), rp, rs, rq, rf, rsd, cp, cs, cq,
                                                 cf, csd, status_word(x.device).data_ptr(), stream_of(x)))
            return
        check(lib().nvfp4_quantize_tile(x.data_ptr(), dtype_code(x), x.shape[0], x.shape[1], x.stride(0), x.stride(1),
                                        signs.data_ptr(), ptr(seed_base), rp, rs, rq, rf, rsd, cp, cs, cq, cf, csd,
                                        status_word(x.device).data_ptr(), stream_of(x)))


def quantize(x, signs, mp, kp, sr, rht, seed, given_scale=None, pair=False, seed_base=None):
    """The reference's native `quantize` operator: returns [packed, scales, pts(, packed_t, scales_t)]."""
    if x.dim() != 2 or not x.is_cuda:
        raise RuntimeError("quantize requires a CUDA 2D tensor")
    dev = x.device
    packed = torch.empty((mp, kp // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty((mp // 128 * 32, kp // 64 * 16), dtype=torch.uint8, device=dev)
    pts = given_scale if given_scale is not None else torch.empty((), dtype=torch.float32, device=dev)
    dt = st = None
    if pair:
        dt = torch.empty((kp, mp // 2), dtype=torch.uint8, device=dev)
        st = torch.empty((kp // 128 * 32, mp // 64 * 16), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        check(lib().nvfp4_quantize(x.data_ptr(), dtype_code(x), x.shape[0], x.shape[1], x.stride(0), x.stride(1), mp, kp,
                                   int(sr), int(bool(rht)), int(seed) & 0xFFFFFFFF, signs.data_ptr(), ptr(given_scale),
                                   ptr(seed_base), int(bool(pair)), packed.data_ptr(), scales.data_ptr(),
                                   None if given_scale is not None else pts.data_ptr(), ptr(dt), ptr(st),
                                   scratch(dev).data_ptr(), status_word(dev).data_ptr(), stream_of(x)))
    return [packed, scales, pts, dt, st] if pair else [packed, scales, pts]


def quantize_fp8_weight(w, unit, pts, *, row=True, col=True):
    """Both orientations (or one) of an E4M3 master weight with per-512 units: (d, s, dt, st), None where not asked."""
    m, k = w.shape
    mp, kp = round128(m), round128(k)
    dev = w.device
    d = s = dt = st = None
    if row:
        d = torch.empty((mp, kp // 2), dtype=torch.uint8, device=dev)
        s = torch.empty((mp // 128 * 32, kp // 64 * 16), dtype=torch.uint8, device=dev)
    if col:
        dt = torch.empty((kp, mp // 2), dtype=torch.uint8, device=dev)
        st = torch.empty((kp // 128 * 32, mp // 64 * 16), dtype=torch.uint8, device=dev)
    if not w.is_contiguous():
        raise ValueError("FP8 master weights must be contiguous")
    with torch.cuda.device(dev):
        check(lib().nvfp4_quantize_fp8_weight(w.data_ptr(), unit.data_ptr(), m, k, pts.data_ptr(), ptr(d), ptr(s), ptr(dt), ptr(st),
                                              stream_of(w)))
    return d, s, dt, st


def dequantize(packed, scales, pts, rows, cols, *, hi_first=False, dtype=torch.float32):
    out = torch.empty((rows, cols), dtype=dtype, device=packed.device)
    with torch.cuda.device(packed.device):
        check(lib().nvfp4_dequantize(packed.data_ptr(), scales.data_ptr(), pts.data_ptr(), packed.shape[1] * 2, rows, cols,
                                     int(hi_first), dtype_code(out), out.data_ptr(), out.stride(0), stream_of(packed)))
    return out


_STATUS: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Device int32 that kernels with bounded waits raise on expiry; read it with check_status()."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _STATUS.get(idx)
    if buf is None:
        buf = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[idx] = buf
    return buf


def check_status(device=None) -> None:
    """Synchronising check of the device status words (tests, check_finite, end of a benchmark)."""
    for idx, buf in _STATUS.items():
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        code = int(buf.item())
        if code:
            buf.zero_()
            raise RuntimeError(f"NVFP4 kernel on cuda:{idx} reported status {code} (bounded device-side wait expired)")


GEMM_SINGLE_CTA = 2
_PAIR = os.environ.get("NVFP4_GEMM_PAIR", "1") != "0"   # NVFP4_GEMM_PAIR=0 keeps every GEMM on single-SM tiles


def gemm(a, sfa, pts_a, b, sfb, pts_b, *, rows, cols, out_dtype=torch.bfloat16, bias=None, raw_bf16=True, out=None, pair=None):
    """out[rows, cols] = crop(A @ B.T) * (pts_a * pts_b) (+ bias); a [M, K/2], b [N, K/2] packed payloads."""
    M, N, K = a.shape[0], b.shape[0], a.shape[1] * 2
    if b.shape[1] != a.shape[1]:
        raise ValueError("Packed contraction dimensions do not match")
    if out is None:
        out = torch.empty((rows, cols), dtype=out_dtype, device=a.device)
    with torch.cuda.device(a.device):
        check(lib().nvfp4_gemm(a.data_ptr(), sfa.data_ptr(), ptr(pts_a), b.data_ptr(), sfb.data_ptr(), ptr(pts_b), M, N, K,
                               ptr(bias), dtype_code(bias) if bias is not None else 0, out.data_ptr(), dtype_code(out),
                               out.stride(0), rows, cols, int(bool(raw_bf16)) | (0 if (_PAIR if pair is None else pair) else GEMM_SINGLE_CTA),
                               status_word(a.device).data_ptr(), stream_of(a)))
    return out


def adamw_step(p, master, grad, m, v, ms, vs, *, vbits, mbits, nonlinear_m, state_block, hyper, step, key, grad_kind=None,
               grad_cols=1, grad_stride=1, sa=None, sb=None, extra=None, grad_mul=1.0, tail=None, unit=None, ctrl=None,
               scale_out=None):
    """In-place compressed AdamW on one flat parameter tensor (see nvfp4_adamw_step)."""
    if grad_kind is None:
        grad_kind = 0 if grad.dtype == torch.float32 else 1
    dev = p.device
    with torch.cuda.device(dev):
        check(lib().nvfp4_adamw_step(p.data_ptr(), master, grad.data_ptr(), grad_kind, grad_cols, grad_stride, ptr(sa), ptr(sb),
                                     ptr(extra), float(grad_mul), m.data_ptr(), ptr(v), ms.data_ptr(), vs.data_ptr(), ptr(tail),
                                     ptr(unit), p.numel(), vbits, mbits, int(bool(nonlinear_m)), state_block, hyper["lr"],
                                     hyper["decay"], hyper["b1"], hyper["b2"], hyper["c1"], hyper["c2"], hyper["eps"],
                                     int(step) & 0xFFFFFFFF, int(key) & 0xFFFFFFFF, ptr(ctrl), ptr(scale_out),
                                     scratch(dev).data_ptr(), stream_of(p)))


PREPACK_FORMATS = {(17, 8, 8, False, 512), (17, 8, 8, False, 128), (24, 8, 8, False, 512), (32, 16, 8, False, 512), (17, 4, 4, True, 512)}


def adamw_step_prepack(p, master, grad, m, v, ms, vs, *, pack, vbits, mbits, nonlinear_m, state_block, hyper, step, key, grad_kind=None,
                       grad_cols=1, grad_stride=1, sa=None, sb=None, extra=None, grad_mul=1.0, tail=None, ctrl=None, scale_out=None):
    """nvfp4_adamw_step on a 2-D weight plus the next forward's packings pack = (d, s, dt, st), written by the same launch."""
    if grad_kind is None:
        grad_kind = 0 if grad.dtype == torch.float32 else 1
    dev = p.device
    d, s, dt, st = pack
    with torch.cuda.device(dev):
        check(lib().nvfp4_adamw_step_prepack(p.data_ptr(), master, grad.data_ptr(), grad_kind, grad_cols, grad_stride, ptr(sa), ptr(sb),
                                             ptr(extra), float(grad_mul), m.data_ptr(), ptr(v), ms.data_ptr(), vs.data_ptr(), ptr(tail),
                                             p.shape[0], p.shape[1], vbits, mbits, int(bool(nonlinear_m)), state_block, hyper["lr"],
                                             hyper["decay"], hyper["b1"], hyper["b2"], hyper["c1"], hyper["c2"], hyper["eps"],
                                             int(step) & 0xFFFFFFFF, int(key) & 0xFFFFFFFF, ptr(ctrl), scale_out.data_ptr(),
                                             d.data_ptr(), s.data_ptr(), dt.data_ptr(), st.data_ptr(), scratch(dev).data_ptr(),
                                             status_word(dev).data_ptr(), stream_of(p)))


def adamw_plain(p, grad, m, v, *, hyper, grad_mul=1.0, ctrl=None):
    with torch.cuda.device(p.device):
        check(lib().nvfp4_adamw_plain(p.data_ptr(), grad.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), float(grad_mul),
                                      hyper["lr"], hyper["decay"], hyper["b1"], hyper["b2"], hyper["c1"], hyper["c2"],
                                      hyper["eps"], ptr(ctrl), stream_of(p)))


def split_init(src, master):
    """FP32 tensor -> (head, tail): FP16 head for master 17, BF16 for 16 / 24 (tail only for 24)."""
    hi = torch.empty_like(src, dtype=torch.float16 if master == 17 else torch.bfloat16)
    tail = torch.empty_like(src, dtype=torch.int8) if master == 24 else None
    with torch.cuda.device(src.device):
        check(lib().nvfp4_split_init(src.data_ptr(), src.numel(), master, hi.data_ptr(), ptr(tail), stream_of(src)))
    return hi, tail
