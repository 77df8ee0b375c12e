"""Golden vectors from the reference's CUDA quantiser, executed on the host.

Run once in the build container, where the reference sources are mounted read-only:

    python tests/golden/make_golden_cuda_quant.py /path/to/reference/src

The reference's native quantiser (src/nvfp4_training/_backend/csrc/kernels.cu) needs an SM120 GPU, but its kernels are
ordinary C++ apart from launch syntax, warp shuffles and shared memory.  This script takes the device code of that file
(`input_value`, `block_max`, `uniform24`, `sr_magnitude`, `reduce_input`, `finish_reduce`, `scale_offset`, `emit_group`,
`quant_rows`, `quant_transpose`, `quant_weight_pair`: everything in front of the first host launcher) UNCHANGED from where
it lies, compiles it as host C++ into a temporary directory (nothing of it is written into this repository) and runs
it under a small SIMT emulator:

  * a thread block is executed thread by thread, repeatedly; every `__shfl_*_sync` records the value its thread passes
    in and returns what the source lane passed in at the same call of the PREVIOUS sweep.  Control flow in front of
    the shuffles is uniform, so after d+1 sweeps a chain of d dependent shuffles is exact; sweeps repeat until the
    record has been identical three times, then one more sweep writes the outputs.  `__shared__` arrays are function
    statics, which the same iteration makes consistent (`__syncthreads` is a no-op);
  * the FP8 / FP4 / BF16 conversions are the host implementations of the CUDA toolkit's own headers;
  * compiled with -ffp-contract=off: every FP32 operation rounds once, like the reference's --fmad=false build.

The host part of `quantize_cuda` (padding, the amax launch shape, which kernel serves which strides) is restated in
the harness below after kernels.cu:237-298.  Cases: the shape / stride / rounding matrix of the reference's acceptance
gate (_verification/verify_fast_v2.py:35-76: 128x256, 193x129 transposed, 130x300[::2, ::2], BF16 and FP32, SR x RHT,
seed 173), zeros, a wide dynamic range, a reused tensor scale and the FP32 weight pair.  Results go to
cuda_quant_reference.npz; the CPU oracle and the sm_100a kernels are checked against that file bit for bit.
"""
import ctypes as C
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

SHIM = r"""
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#undef __shared__
#define __shared__ static
#undef __global__
#define __global__
namespace sim {
struct Idx { unsigned x, y, z; };
static Idx tid, bid, bdim, gdim;
static std::vector<std::vector<uint32_t>> prev, cur;
static size_t call;
template <class T> static T exchange(T v, int src) {
    static_assert(sizeof(T) == 4, "32-bit shuffles only");
    uint32_t bits; std::memcpy(&bits, &v, 4);
    auto& mine = cur[tid.x];
    if (mine.size() <= call) mine.resize(call + 1);
    mine[call] = bits;
    uint32_t got = bits;
    if (src != (int)tid.x) got = call < prev[src].size() ? prev[src][call] : 0u;
    ++call;
    T r; std::memcpy(&r, &got, 4); return r;
}
template <class F> static void run_block(int threads, F body) {
    prev.assign(threads, {});
    int same = 0;
    for (int sweep = 0; sweep < 200; ++sweep) {
        cur.assign(threads, {});
        for (int t = 0; t < threads; ++t) { tid.x = t; call = 0; body(); }
        const bool equal = cur == prev;
        prev.swap(cur);
        if (same >= 3) return;          // this sweep ran on a record that had already repeated three times
        same = equal ? same + 1 : 0;
    }
    std::abort();
}
}  // namespace sim
#define threadIdx sim::tid
#define blockIdx sim::bid
#define blockDim sim::bdim
#define gridDim sim::gdim
template <class T> static T __shfl_xor_sync(unsigned, T v, int d, int width = 32) {
    const int t = sim::tid.x;
    return sim::exchange(v, (t & ~(width - 1)) | ((t ^ d) & (width - 1)));
}
template <class T> static T __shfl_down_sync(unsigned, T v, int d, int width = 32) {
    const int t = sim::tid.x, lane = t & (width - 1);
    return sim::exchange(v, lane + d < width ? t + d : t);
}
static inline void __syncthreads() {}
"""

HARNESS = r"""
static int64_t round128(int64_t n) { return (n + 127) / 128 * 128; }
template <class F> static void launch(unsigned gx, unsigned gy, F body) {
    sim::gdim = {gx, gy, 1}; sim::bdim = {THREADS, 1, 1};
    for (unsigned y = 0; y < gy; ++y) for (unsigned x = 0; x < gx; ++x) { sim::bid = {x, y, 0}; sim::run_block(THREADS, body); }
}
template <bool F32, bool SR, bool RHT>
static void quant(const void* x, uint8_t* d, uint8_t* s, const float* p, const float* sg, int64_t m, int64_t k, int64_t mp,
                  int64_t kp, int64_t s0, int64_t s1, uint32_t seed) {
    if (s0 == 1 && s1 != 1) launch(kp / 64, mp / 32, [&] { quant_transpose<F32, SR, RHT>(x, d, s, p, sg, m, k, mp, kp, s0, s1, seed); });
    else launch(kp / 128, mp / 16, [&] { quant_rows<F32, SR, RHT>(x, d, s, p, sg, m, k, mp, kp, s0, s1, seed); });
}
template <bool F32>
static void select(const void* x, uint8_t* d, uint8_t* s, const float* p, const float* sg, int64_t m, int64_t k, int64_t mp,
                   int64_t kp, int64_t s0, int64_t s1, uint32_t seed, bool sr, bool rht) {
    if (sr && rht) quant<F32, true, true>(x, d, s, p, sg, m, k, mp, kp, s0, s1, seed);
    else if (sr) quant<F32, true, false>(x, d, s, p, sg, m, k, mp, kp, s0, s1, seed);
    else if (rht) quant<F32, false, true>(x, d, s, p, sg, m, k, mp, kp, s0, s1, seed);
    else quant<F32, false, false>(x, d, s, p, sg, m, k, mp, kp, s0, s1, seed);
}
template <bool F32>
static void tensor_scale(const void* x, float* pts, int64_t m, int64_t k, int64_t s0, int64_t s1, bool contiguous, float factor) {
    int count = (int)std::min<int64_t>((m * k + 1023) / 1024, 1024);
    count = std::max(1, count);
    std::vector<float> partial(count);
    float* dst = count == 1 ? pts : partial.data();
    const bool dense = contiguous || (s0 == 1 && s1 == m);
    launch(count, 1, [&] { reduce_input<F32>(x, dst, m, k, s0, s1, dense, count == 1, factor); });
    if (count > 1) launch(1, 1, [&] { finish_reduce(partial.data(), pts, count, factor); });
}
extern "C" void ref_quantize(const void* x, int f32, int64_t m, int64_t k, int64_t s0, int64_t s1, int contiguous, int sr, int rht,
                             uint32_t seed, const float* signs, float* pts, int given, uint8_t* packed, uint8_t* scales) {
    const int64_t mp = round128(m), kp = round128(k);
    if (!given) {
        if (f32) tensor_scale<true>(x, pts, m, k, s0, s1, contiguous, rht ? 4.f : 1.f);
        else tensor_scale<false>(x, pts, m, k, s0, s1, contiguous, rht ? 4.f : 1.f);
    }
    if (f32) select<true>(x, packed, scales, pts, signs, m, k, mp, kp, s0, s1, seed, sr, rht);
    else select<false>(x, packed, scales, pts, signs, m, k, mp, kp, s0, s1, seed, sr, rht);
}
extern "C" void ref_weight_pair(const float* x, int m, int k, const float* pts, uint8_t* data, uint8_t* scale, uint8_t* dt, uint8_t* st) {
    const int mp = (int)round128(m), kp = (int)round128(k);
    launch(kp / 64, mp / 32, [&] { quant_weight_pair(x, data, scale, dt, st, pts, m, k, mp, kp); });
}
"""


def device_code(src_root: Path) -> str:
    text = (src_root / "nvfp4_training" / "_backend" / "csrc" / "kernels.cu").read_text()
    start = text.index("constexpr int THREADS")
    stop = text.index("template<bool F32,bool SR,bool RHT>\nvoid launch_quant")
    return text[start:stop]


def build(src_root: Path, tmp: Path):
    cpp = tmp / "ref_quant.cpp"
    cpp.write_text(SHIM + device_code(src_root) + HARNESS)
    so = tmp / "ref_quant.so"
    subprocess.run(["/usr/bin/g++", "-O1", "-std=c++17", "-ffp-contract=off", "-fno-fast-math", "-I/usr/local/cuda/include",
                    "-shared", "-fPIC", "-o", str(so), str(cpp)], check=True)
    L = C.CDLL(str(so))
    L.ref_quantize.restype = None
    L.ref_quantize.argtypes = ([C.c_void_p, C.c_int] + [C.c_int64] * 4 + [C.c_int] * 3 + [C.c_uint32, C.c_void_p, C.c_void_p, C.c_int,
                               C.c_void_p, C.c_void_p])
    L.ref_weight_pair.restype = None
    L.ref_weight_pair.argtypes = [C.c_void_p, C.c_int, C.c_int] + [C.c_void_p] * 5
    return L


def round128(n):
    return (n + 127) // 128 * 128


def view_of(base: torch.Tensor, kind: int) -> torch.Tensor:
    """kind 0: the tensor itself; 1: its transpose (a view); 2: every second row and column."""
    return base if kind == 0 else base.t() if kind == 1 else base[::2, ::2]


def run_quantize(L, x: torch.Tensor, signs: np.ndarray, sr, rht, seed, given=None):
    m, k = x.shape
    mp, kp = round128(m), round128(k)
    packed = np.zeros((mp, kp // 2), dtype=np.uint8)
    scales = np.zeros((mp // 128 * 32, kp // 64 * 16), dtype=np.uint8)
    pts = np.array([given if given is not None else 0.0], dtype=np.float32)
    L.ref_quantize(x.data_ptr(), int(x.dtype == torch.float32), m, k, x.stride(0), x.stride(1), int(x.is_contiguous()), int(sr),
                   int(rht), seed, signs.ctypes.data, pts.ctypes.data, int(given is not None), packed.ctypes.data, scales.ctypes.data)
    return packed, scales, pts


def store(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).numpy().view(np.uint16).copy() if t.dtype == torch.bfloat16 else t.numpy().copy()


def main():
    src_root = Path(sys.argv[1])
    gen = torch.Generator().manual_seed(9107)
    sg = torch.Generator(device="cpu").manual_seed(1)
    signs = (torch.randint(0, 2, (16,), generator=sg).float() * 2 - 1).numpy().copy()
    out = {"signs": signs}
    names = []
    with tempfile.TemporaryDirectory() as tmp:
        L = build(src_root, Path(tmp))

        def case(name, base_name, base, kind, sr, rht, seed, given=None):
            x = view_of(base, kind)
            p, s, t = run_quantize(L, x, signs, sr, rht, seed, given)
            out[f"base_{base_name}"] = store(base)
            out[f"{name}_base"] = np.array(base_name)
            out[f"{name}_meta"] = np.array([kind, int(base.dtype == torch.bfloat16), int(sr), int(rht), seed, int(given is not None)],
                                           dtype=np.int64)
            out[f"{name}_data"], out[f"{name}_scale"], out[f"{name}_pts"] = p, s, t
            names.append(name)

        for dt, dtype in (("bf16", torch.bfloat16), ("f32", torch.float32)):
            bases = {"aligned": (torch.randn(128, 256, generator=gen).to(dtype), 0),
                     "transposed": (torch.randn(193, 129, generator=gen).to(dtype), 1),
                     "strided": (torch.randn(130, 300, generator=gen).to(dtype), 2)}
            for label, (base, kind) in bases.items():
                for sr, rht in ((False, False), (True, False), (False, True), (True, True)):
                    case(f"{dt}_{label}_sr{int(sr)}_rht{int(rht)}", f"{dt}_{label}", base, kind, sr, rht, 173)
        case("zeros", "zeros", torch.zeros(17, 35), 0, True, True, 0)
        # magnitudes spread over 2^-20 .. 2^8 so that the FP32 butterfly rounds and the block-scale clamps are reached
        wide = torch.randn(64, 160, generator=gen) * torch.exp2(torch.randint(-20, 9, (64, 160), generator=gen).float())
        case("wide_rht", "wide_bf16", wide.bfloat16(), 0, False, True, 5)
        case("wide_sr", "wide_f32", wide, 0, True, False, 6)
        case("wide_t_sr_rht", "wide_bf16", wide.bfloat16(), 1, True, True, 7)
        case("given_scale", "given", torch.randn(40, 48, generator=gen).bfloat16(), 0, True, True, 4242, given=0.00371)
        case("seed_wrap", "wrap", torch.randn(33, 140, generator=gen).bfloat16(), 0, True, False, 0xFFFFFFF0)
        w = torch.randn(160, 200, generator=gen) * 0.02
        mp, kp = round128(160), round128(200)
        pts = np.array([np.float32(max(float(w.bfloat16().float().abs().max()), 1e-12)) * np.float32(1.0 / 2688.0)], dtype=np.float32)
        d, s = np.zeros((mp, kp // 2), np.uint8), np.zeros((mp // 128 * 32, kp // 64 * 16), np.uint8)
        dt_, st = np.zeros((kp, mp // 2), np.uint8), np.zeros((kp // 128 * 32, mp // 64 * 16), np.uint8)
        L.ref_weight_pair(w.data_ptr(), 160, 200, pts.ctypes.data, d.ctypes.data, s.ctypes.data, dt_.ctypes.data, st.ctypes.data)
        out.update(pair_w=w.numpy().copy(), pair_pts=pts, pair_data=d, pair_scale=s, pair_data_t=dt_, pair_scale_t=st)
    out["names"] = np.array(names)
    np.savez_compressed(HERE / "cuda_quant_reference.npz", **out)
    print("wrote", HERE / "cuda_quant_reference.npz", len(names), "quantise cases + weight pair")


if __name__ == "__main__":
    main()
