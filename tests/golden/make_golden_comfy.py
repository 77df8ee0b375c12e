"""Golden vectors for the scalar arithmetic of the packed-checkpoint LoRA backend.

Run once in the build container, where the reference sources are mounted read-only:

    python tests/golden/make_golden_comfy.py /path/to/reference/src

The reference keeps this backend's device code as one CUDA C source string (src/precision_lora/_packed_cuda.py:13-164)
that it compiles with NVRTC at run time.  The kernels need a GPU, but the scalar device functions in front of them
(BF16 decode/round, E4M3 decode/encode, E2M1 decode/encode with stochastic rounding, the integer mixer, the scale
swizzle) are plain C once three CUDA intrinsics are supplied.  This script takes that part of the string from the
reference file where it lies, compiles it as host C++ into a temporary directory (nothing of it is written into this
repository), evaluates the functions on the inputs generated below and stores inputs and outputs in
comfy_scalar_reference.npz.  The CPU oracle (oracle/comfy_oracle.c) is then checked against the file bit for bit.
"""
import ctypes as C
import importlib.util
import re
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

SHIM = r"""
#include <cmath>
#include <cstring>
#include <cstdint>
#define __device__ static
static inline float __uint_as_float(unsigned u) { float f; std::memcpy(&f, &u, 4); return f; }
static inline unsigned __float_as_uint(float f) { unsigned u; std::memcpy(&u, &f, 4); return u; }
static inline int __float2int_rn(float x) { return (int)std::lrintf(x); }
using std::signbit;
"""

WRAPPERS = r"""
extern "C" {
float ref_bf(unsigned short x) { return bf(x); }
unsigned short ref_rb(float x) { return rb(x); }
float ref_f8(unsigned char x) { return f8(x); }
unsigned char ref_rf8(float v) { return rf8(v); }
float ref_f4(int c) { return f4(c); }
unsigned ref_mix(unsigned x) { return mix(x); }
unsigned char ref_rf4(float v, unsigned rng, int sr) { return rf4(v, rng, sr); }
long long ref_swizzle(int r, int b, int k) { return swizzle(r, b, k); }
}
"""


def reference_scalars(src_root: Path) -> str:
    spec = importlib.util.spec_from_file_location("_ref_packed_cuda", src_root / "precision_lora" / "_packed_cuda.py")
    text = spec.loader.get_source("_ref_packed_cuda")
    source = re.search(r"SOURCE=r'''(.*?)'''", text, re.S).group(1)
    head = source[: source.index('extern "C" __global__')]
    # the hardware E2M1 pair conversion is inline PTX; it is pinned through the quantiser fixtures instead
    head = re.sub(r"__device__ unsigned pack_rne\(.*?\n\}\n", "", head, flags=re.S)
    return head


def inputs(rng: np.random.Generator) -> dict:
    finite = rng.integers(0, 2**32, 40000, dtype=np.uint64).astype(np.uint32)
    finite = finite[((finite >> 23) & 255) != 255]
    f8_values = np.array([0.0] + [2.0 ** e * (1 + m / 8) for e in range(-6, 9) for m in range(8)] +
                         [m * 2.0 ** -9 for m in range(8)], dtype=np.float64)
    mids = (f8_values[:, None] + f8_values[None, :]).ravel() / 2
    rf8_in = np.concatenate([np.exp2(rng.uniform(-13, 9.5, 30000)), f8_values, mids[:4000], [447.9, 448, 449, 1e9, 1e-30, -1.0]])
    levels = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], dtype=np.float64)
    lv_mid = np.concatenate([levels, (levels[1:] + levels[:-1]) / 2, [6.5, 7, 100]])
    rf4_v = np.concatenate([rng.uniform(-7, 7, 30000), lv_mid, -lv_mid, [-0.0]]).astype(np.float32)
    return dict(rb_in=finite.view(np.float32), bf_in=rng.integers(0, 2**16, 4000).astype(np.uint16),
                f8_in=np.arange(256, dtype=np.uint8), rf8_in=rf8_in.astype(np.float32), f4_in=np.arange(16, dtype=np.int32),
                mix_in=rng.integers(0, 2**32, 20000, dtype=np.uint64).astype(np.uint32), rf4_v=rf4_v,
                rf4_rng=rng.integers(0, 2**32, rf4_v.size, dtype=np.uint64).astype(np.uint32),
                sw_r=rng.integers(0, 5000, 4000).astype(np.int32), sw_b=rng.integers(0, 800, 4000).astype(np.int32),
                sw_k=(rng.integers(1, 800, 4000) * 16).astype(np.int32))


def main():
    src_root = Path(sys.argv[1])
    with tempfile.TemporaryDirectory() as tmp:
        cpp = Path(tmp) / "scalars.cpp"
        cpp.write_text(SHIM + reference_scalars(src_root) + WRAPPERS)
        so = Path(tmp) / "scalars.so"
        subprocess.run(["/usr/bin/g++", "-O1", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC", "-o", str(so), str(cpp)],
                       check=True)
        L = C.CDLL(str(so))
        L.ref_bf.restype = C.c_float; L.ref_bf.argtypes = [C.c_ushort]
        L.ref_rb.restype = C.c_ushort; L.ref_rb.argtypes = [C.c_float]
        L.ref_f8.restype = C.c_float; L.ref_f8.argtypes = [C.c_ubyte]
        L.ref_rf8.restype = C.c_ubyte; L.ref_rf8.argtypes = [C.c_float]
        L.ref_f4.restype = C.c_float; L.ref_f4.argtypes = [C.c_int]
        L.ref_mix.restype = C.c_uint; L.ref_mix.argtypes = [C.c_uint]
        L.ref_rf4.restype = C.c_ubyte; L.ref_rf4.argtypes = [C.c_float, C.c_uint, C.c_int]
        L.ref_swizzle.restype = C.c_longlong; L.ref_swizzle.argtypes = [C.c_int] * 3
        d = inputs(np.random.default_rng(20240607))
        out = dict(d)
        out["bf_out"] = np.array([L.ref_bf(int(v)) for v in d["bf_in"]], dtype=np.float32).view(np.uint32)
        out["rb_out"] = np.array([L.ref_rb(float(v)) for v in d["rb_in"]], dtype=np.uint16)
        out["f8_out"] = np.array([L.ref_f8(int(v)) for v in d["f8_in"]], dtype=np.float32)
        out["rf8_out"] = np.array([L.ref_rf8(float(v)) for v in d["rf8_in"]], dtype=np.uint8)
        out["f4_out"] = np.array([L.ref_f4(int(v)) for v in d["f4_in"]], dtype=np.float32)
        out["mix_out"] = np.array([L.ref_mix(int(v)) for v in d["mix_in"]], dtype=np.uint32)
        for sr in (0, 1):
            out[f"rf4_out_sr{sr}"] = np.array([L.ref_rf4(float(v), int(r), sr) for v, r in zip(d["rf4_v"], d["rf4_rng"])],
                                              dtype=np.uint8)
        out["sw_out"] = np.array([L.ref_swizzle(int(r), int(b), int(k)) for r, b, k in zip(d["sw_r"], d["sw_b"], d["sw_k"])],
                                 dtype=np.int64)
        out["rb_in"] = d["rb_in"].view(np.uint32)   # bit patterns: NaN-free but keeps -0 and denormals exact
    np.savez_compressed(HERE / "comfy_scalar_reference.npz", **out)
    print("wrote", HERE / "comfy_scalar_reference.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
