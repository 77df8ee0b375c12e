// nvcc-flags: --fmad=false
// Compressed AdamW step for sm_100a: ONE kernel decodes the block-scaled low-precision moments and the
// master weight, applies AdamW, re-encodes everything (stochastic rounding where the format asks for it),
// and reduces the amax of the BF16-rounded new weight to the tensor scale the next forward will use.
//
// This file is compiled without FMA contraction: each * + - / below is one IEEE FP32 rounding, which is the
// arithmetic the storage formats were defined with.  sqrtf and / are the correctly rounded forms.
//
// The kernel is latency- and issue-bound, not HBM-bound (about 150 instructions per element with square-root and division
// chains), so it is compiled for four CTAs per SM (64 registers, a few spilled words): measured 0.286 -> 0.222 ms on a
// 4096 x 8192 weight against the 107-register build.  A variant with 8 elements per lane (no spills, two warps per
// 512-element block through shared memory) measured 0.268 ms and was dropped.
//
// Work split: a warp owns 512 consecutive elements, lane l the 16 elements [16 l, 16 l + 16).  State blocks
// (512, 256, 128 or 64 elements) therefore cover 32, 16, 8 or 4 adjacent lanes and their maxima are plain
// segmented shuffles: no shared memory, no block barrier on the data path.
#include "pack_tile.cuh"

#include <algorithm>
#include <cstdlib>

#ifndef ADAM_MIN_BLOCKS
#define ADAM_MIN_BLOCKS 4   // resident CTAs per SM the update kernel is compiled for (64 registers per thread)
#endif

namespace nvfp4 {

struct AdamArgs {
    void* p; const void* grad; const float* extra; void* m; void* v; float* ms; float* vs; int8_t* tail; float* unit;
    const float* sa; const float* sb; const float* ctrl; float* scale_out; unsigned int* scratch;
    int64_t n, grad_cols, grad_stride;
    int grad_kind;  // 0 FP32, 1 BF16, 2 raw BF16 GEMM output times bf16(sa*sb)
    float lr, decay, b1, b2, c1, c2, eps, grad_mul;
    uint32_t step, key;
};

__device__ __forceinline__ uint32_t adam_bits(uint32_t index, uint32_t step, uint32_t key) {
    uint32_t z = index + step * 0x9e3779b9u + key;
    z = (z ^ (z >> 16)) * 0x7feb352du;
    z = (z ^ (z >> 15)) * 0x846ca68bu;
    return z ^ (z >> 16);
}
__device__ __forceinline__ int signed_tail(float x, uint16_t hi) {
    const uint32_t upper = static_cast<uint32_t>(hi) << 16;
    const int delta = static_cast<int>(__float_as_uint(x) - upper);
    const int rounded = (delta + 127 + ((delta >> 8) & 1)) >> 8;
    return max(-128, min(127, rounded));
}
__device__ __forceinline__ float seg_max(float x, int lanes) {  // max over aligned groups of `lanes` lanes
    for (int d = 1; d < lanes; d <<= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, d));
    return x;
}
__device__ __forceinline__ uint8_t e4m3_sr(float x, uint32_t bits) {
    const uint32_t raw = __float_as_uint(x);
    const float normal = __uint_as_float((raw + (bits & 0xfffffu)) & 0xfff00000u);
    const float mag = fabsf(x) * 512.f;
    const float low = floorf(mag);
    const float sub = (low + static_cast<float>((static_cast<float>(bits & 0xfffffu) / 1048576.f) < (mag - low))) / 512.f;
    const float val = fabsf(x) < .015625f ? (x < 0.f ? 0.f - sub : sub) : normal;
    if (!(fabsf(x) <= 448.f)) return static_cast<uint8_t>(0x7f | ((raw >> 24) & 0x80u));
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(val, __NV_SATFINITE, __NV_E4M3));
}

// Exact small-integer -> float moves that stay off the quarter-rate conversion pipe: an unsigned integer below 2^23
// dropped into the mantissa of 2^23 is the float 2^23 + n.
__device__ __forceinline__ float byte_as_float(uint32_t word, uint32_t selector) {   // selector 0x7650 + byte index
    return __uint_as_float(__byte_perm(word, 0x4B000000u, selector)) - 8388608.f;
}
__device__ __forceinline__ float u16_as_float(uint32_t x) { return __uint_as_float(0x4B000000u | x) - 8388608.f; }

// u < ((z - lo) * (z + lo)) / (2 lo + 1) for a 16-bit uniform u = k / 65536, without the division: with A the rounded
// numerator and D = 2 lo + 1, RN(A / D) > u exactly when A - D u > D * (half an ulp of u), and near that boundary the
// left side is exact in one FMA.  Enumerated against the division over every float z of [0, 255] and the values of k
// around the turning point (tests/exact_threshold.c).
__device__ __forceinline__ bool rounds_up(float z, float lo, float u) {
    const float A = __fmul_rn(z - lo, z + lo);
    const float D = __fmaf_rn(2.f, lo, 1.f);
    const int half_ulp = static_cast<int>(__float_as_uint(u) & 0x7f800000u) - (24 << 23);   // negative for u = 0
    return __fmaf_rn(-D, u, A) > __fmul_rn(D, __int_as_float(max(half_ulp, 0)));
}

// 16 consecutive items of T starting at element i0; vector loads when the run is complete and aligned.
template <typename T>
__device__ __forceinline__ void load16(const T* base, int64_t i0, int64_t n, T (&out)[16], T fill) {
    constexpr int BYTES = 16 * sizeof(T);
    if (i0 + 16 <= n && (reinterpret_cast<uintptr_t>(base + i0) & 15) == 0) {
        uint4 tmp[BYTES / 16];
#pragma unroll
        for (int j = 0; j < BYTES / 16; ++j) tmp[j] = reinterpret_cast<const uint4*>(base + i0)[j];
        memcpy(out, tmp, BYTES);
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) out[j] = (i0 + j < n) ? base[i0 + j] : fill;
    }
}
template <typename T>
__device__ __forceinline__ void store16(T* base, int64_t i0, int64_t n, const T (&in)[16]) {
    constexpr int BYTES = 16 * sizeof(T);
    if (i0 + 16 <= n && (reinterpret_cast<uintptr_t>(base + i0) & 15) == 0) {
        uint4 tmp[BYTES / 16];
        memcpy(tmp, in, BYTES);
#pragma unroll
        for (int j = 0; j < BYTES / 16; ++j) reinterpret_cast<uint4*>(base + i0)[j] = tmp[j];
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) if (i0 + j < n) base[i0 + j] = in[j];
    }
}

// The update of one chunk of 4096 elements by a CTA of 256 threads; returns this lane's share of max |bf16(new weight)|.
template <int MASTER, int VB, bool M4, bool NL, int B>
__device__ __forceinline__ float adam_chunk(const AdamArgs& a, int64_t chunk, float c1, float c2, uint32_t step) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t i0 = (chunk * 8 + warp) * 512 + lane * 16;
    const int64_t n = a.n;
    const bool any = i0 < n;
    const int64_t blk = i0 / B;
    constexpr int LANES_B = B / 16;
    const float one_b1 = 1.f - a.b1, one_b2 = 1.f - a.b2, lrc1 = a.lr * c1;

    float p[16], g[16], m[16], v[16];
    // ---- master decode ----
    float unit = 1.f;
    if constexpr (MASTER == 32) {
        load16(static_cast<const float*>(a.p), i0, n, p, 0.f);
    } else if constexpr (MASTER == 8) {
        uint8_t raw[16];
        load16(static_cast<const uint8_t*>(a.p), i0, n, raw, uint8_t(0));
        unit = any ? a.unit[i0 / 512] : 1.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) p[j] = e4m3_to_float(raw[j]) * unit;
    } else {
        uint16_t raw[16];
        load16(static_cast<const uint16_t*>(a.p), i0, n, raw, uint16_t(0));
        if constexpr (MASTER == 24) {
            int8_t tl[16];
            load16(a.tail, i0, n, tl, int8_t(0));
#pragma unroll
            for (int j = 0; j < 16; ++j)
                p[j] = __uint_as_float((static_cast<uint32_t>(raw[j]) << 16) + static_cast<uint32_t>(static_cast<int>(tl[j]) * 256));
        } else if constexpr (MASTER == 17) {
#pragma unroll
            for (int j = 0; j < 16; ++j) p[j] = __half2float(__ushort_as_half(raw[j]));
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) p[j] = bf16_value(raw[j]);
        }
    }
    // ---- gradient decode ----
    if (a.grad_kind == 0) {
        load16(static_cast<const float*>(a.grad), i0, n, g, 0.f);
    } else {
        uint16_t raw[16];
        if (a.grad_kind == 1 || a.grad_cols == a.grad_stride) {
            load16(static_cast<const uint16_t*>(a.grad), i0, n, raw, uint16_t(0));
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int64_t i = i0 + j;
                raw[j] = i < n ? static_cast<const uint16_t*>(a.grad)[(i / a.grad_cols) * a.grad_stride + i % a.grad_cols] : uint16_t(0);
            }
        }
        if (a.grad_kind == 2) {
            const float alpha = bf16_value(bf16_bits(a.sa[0] * a.sb[0]));
#pragma unroll
            for (int j = 0; j < 16; ++j) g[j] = bf16_value(bf16_bits(bf16_value(raw[j]) * alpha));
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) g[j] = bf16_value(raw[j]);
        }
    }
    if (a.extra) {
        float e[16];
        load16(a.extra, i0, n, e, 0.f);
#pragma unroll
        for (int j = 0; j < 16; ++j) g[j] += e[j];
    }
    if (a.grad_mul != 1.f) {
#pragma unroll
        for (int j = 0; j < 16; ++j) g[j] *= a.grad_mul;
    }
    // ---- moment decode ----
    uint8_t nib[16];  // M4 && VB == 4: one byte per element (m low nibble, v high nibble)
    if constexpr (M4) {
        const float s = any ? a.ms[i0 / 64] : 0.f;
        if constexpr (VB == 4) {
            load16(static_cast<const uint8_t*>(a.m), i0, n, nib, uint8_t(7));
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                float c = static_cast<float>(static_cast<int>(nib[j] & 15) - 7);
                if constexpr (NL) c = c * fabsf(c);
                m[j] = (i0 + j < n) ? c * s : 0.f;
            }
        } else {
            uint8_t pk[8] = {};
            const int64_t pn = (n + 1) / 2;
            if (i0 / 2 + 8 <= pn) memcpy(pk, static_cast<const uint8_t*>(a.m) + i0 / 2, 8);
            else for (int j = 0; j < 8; ++j) pk[j] = (i0 / 2 + j < pn) ? static_cast<const uint8_t*>(a.m)[i0 / 2 + j] : 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                float c = static_cast<float>(static_cast<int>((j & 1) ? (pk[j >> 1] >> 4) : (pk[j >> 1] & 15)) - 7);
                if constexpr (NL) c = c * fabsf(c);
                m[j] = (i0 + j < n) ? c * s : 0.f;
            }
        }
    } else {
        int8_t raw[16];
        load16(static_cast<const int8_t*>(a.m), i0, n, raw, int8_t(0));
        uint32_t w[4];
        memcpy(w, raw, 16);
        const float s = any ? a.ms[blk] : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j)   // int8 -> float: (2^23 + (byte ^ 0x80)) - (2^23 + 128), one exact subtraction
            m[j] = (__uint_as_float(__byte_perm(w[j >> 2] ^ 0x80808080u, 0x4B000000u, 0x7650u + (j & 3))) - 8388736.f) * s;
    }
    if constexpr (VB == 4) {
        const float s = any ? a.vs[i0 / 64] : 0.f;
        if constexpr (M4) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = (i0 + j < n) ? static_cast<float>(nib[j] >> 4) * s : 0.f;
        } else {
            uint8_t pk[8] = {};
            const int64_t pn = (n + 1) / 2;
            if (i0 / 2 + 8 <= pn) memcpy(pk, static_cast<const uint8_t*>(a.v) + i0 / 2, 8);
            else for (int j = 0; j < 8; ++j) pk[j] = (i0 / 2 + j < pn) ? static_cast<const uint8_t*>(a.v)[i0 / 2 + j] : 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = static_cast<float>((j & 1) ? (pk[j >> 1] >> 4) : (pk[j >> 1] & 15)) * s;
        }
    } else if constexpr (VB == 8) {
        uint8_t raw[16];
        load16(static_cast<const uint8_t*>(a.v), i0, n, raw, uint8_t(0));
        uint32_t w[4];
        memcpy(w, raw, 16);
        const float s = any ? a.vs[blk] : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = byte_as_float(w[j >> 2], 0x7650u + (j & 3)) * s;
    } else {
        uint16_t raw[16];
        load16(static_cast<const uint16_t*>(a.v), i0, n, raw, uint16_t(0));
        const float s = any ? a.vs[blk] : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __half2float(__ushort_as_half(raw[j])) * s;
    }
    if constexpr (VB < 16) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = v[j] * v[j];
    }
    // ---- AdamW ----
    float root[16], upd[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float t1 = a.b1 * m[j], t2 = one_b1 * g[j];
        m[j] = t1 + t2;
        const float t3 = a.b2 * v[j], t4 = (one_b2 * g[j]) * g[j];
        v[j] = t3 + t4;
        root[j] = sqrtf(v[j]);
        const float decayed = p[j] * a.decay;
        upd[j] = decayed - (lrc1 * m[j]) / (root[j] * c2 + a.eps);
    }
    // ---- master store; hi = the BF16 value the next forward will quantise ----
    float amax = 0.f;
    if constexpr (MASTER == 32) {
        store16(static_cast<float*>(a.p), i0, n, upd);
#pragma unroll
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(bf16_value(bf16_bits(upd[j]))));   // padding updates to zero
    } else if constexpr (MASTER == 8) {
        float peak = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) if (i0 + j < n) peak = fmaxf(peak, fabsf(upd[j]));
        peak = seg_max(peak, 32);
        const bool grow = (peak > 448.f * unit) && (peak < INFINITY);
        if (grow) {
            const float raised = exp2f(floorf(log2f(fmaxf(peak, 1.e-30f))) - 7.f);
            unit = fmaxf(unit, raised);
            if (lane == 0) a.unit[i0 / 512] = unit;
        }
        uint8_t out[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            out[j] = e4m3_sr(upd[j] / unit, adam_bits(static_cast<uint32_t>(i0 + j), step, a.key + 198743u));
            if (i0 + j < n) amax = fmaxf(amax, fabsf(bf16_value(bf16_bits(e4m3_to_float(out[j]) * unit))));
        }
        store16(static_cast<uint8_t*>(a.p), i0, n, out);
    } else {
        uint16_t out[16];
        [[maybe_unused]] int8_t tl[16];
        // FP16 masters: weights in the subnormal range of FP16 take their own rounding; one test per lane keeps the branch
        // out of the element loop
        [[maybe_unused]] bool tiny_any = false;
        if constexpr (MASTER == 17) {
            float least = 1.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) least = fminf(least, fabsf(upd[j]));
            tiny_any = least < 0.00006103515625f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float u = upd[j];
            float hi;
            if constexpr (MASTER == 24) {
                out[j] = bf16_bits(u);
                tl[j] = static_cast<int8_t>(signed_tail(u, out[j]));
                hi = bf16_value(out[j]);
            } else if constexpr (MASTER == 17) {
                const uint32_t rnd = adam_bits(static_cast<uint32_t>(i0 + j), step, a.key);
                const uint32_t raw = __float_as_uint(u);
                uint16_t half = __half_as_ushort(__float2half_rn(__uint_as_float((raw + (rnd & 8191u)) & 0xffffe000u)));
                if (tiny_any && fabsf(u) < 0.00006103515625f) {
                    const float mag = fabsf(u) * 16777216.f;
                    const float fl = floorf(mag);
                    const float sub = fl + static_cast<float>((static_cast<float>(rnd & 65535u) / 65536.f) < (mag - fl));
                    half = static_cast<uint16_t>(static_cast<uint32_t>(sub) | ((raw >> 16) & 32768u));
                }
                out[j] = half;
                hi = bf16_value(bf16_bits(__half2float(__ushort_as_half(half))));
            } else {
                const uint32_t rnd = adam_bits(static_cast<uint32_t>(i0 + j), step, a.key);
                out[j] = static_cast<uint16_t>((__float_as_uint(u) + (rnd & 65535u)) >> 16);
                hi = bf16_value(out[j]);
            }
            amax = fmaxf(amax, fabsf(hi));   // elements past the end were loaded as zeros and update to an exact zero
        }
        store16(static_cast<uint16_t*>(a.p), i0, n, out);
        if constexpr (MASTER == 24) store16(a.tail, i0, n, tl);
    }
    // ---- momentum store ----
    [[maybe_unused]] uint32_t mcode[16];
    if constexpr (M4) {
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) mx = fmaxf(mx, fabsf(m[j]));
        mx = seg_max(mx, 4);
        const float sc = NL ? fmaxf(mx / 49.f, 1.e-30f) : fmaxf(mx / 7.f, 1.e-30f);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float norm, fl, prob;
            if constexpr (NL) {
                norm = fminf(7.f, sqrtf(fabsf(m[j]) / sc));
                fl = floorf(norm);
                prob = (norm - fl) * (norm + fl) / (2.f * fl + 1.f);
            } else {
                norm = fmaxf(-7.f, fminf(7.f, m[j] / sc));
                fl = floorf(norm);
                prob = norm - fl;
            }
            const uint32_t rb = adam_bits(static_cast<uint32_t>(i0 + j), step, a.key + 7131821u);
            const float uu = static_cast<float>(rb >> 8) * (1.f / 16777216.f);
            int mc = static_cast<int>(fl + static_cast<float>(uu < prob));
            if constexpr (NL) { if (m[j] < 0.f) mc = -mc; }
            mcode[j] = static_cast<uint32_t>(mc + 7);
        }
        if (any && (lane & 3) == 0) a.ms[i0 / 64] = sc;
        if constexpr (VB != 4) {
            uint8_t pk[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) pk[j] = static_cast<uint8_t>(mcode[2 * j] | (mcode[2 * j + 1] << 4));
            const int64_t pn = (n + 1) / 2;
            if (i0 / 2 + 8 <= pn) memcpy(static_cast<uint8_t*>(a.m) + i0 / 2, pk, 8);
            else for (int j = 0; j < 8; ++j) if (i0 / 2 + j < pn) static_cast<uint8_t*>(a.m)[i0 / 2 + j] = pk[j];
        }
    } else {
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) mx = fmaxf(mx, fabsf(m[j]));
        mx = seg_max(mx, LANES_B);
        const float sc = fmaxf(mx / 127.f, 1.e-30f);
        int8_t out[16];
        // |m| <= 127 sc; a quotient under 2^-43 rounds to code 0 whatever its last bits are
        const SharedDivisor by_sc = shared_divisor(sc);
        if (by_sc.safe) {
#pragma unroll
            for (int j = 0; j < 16; ++j) out[j] = static_cast<int8_t>(max(-127, min(127, __float2int_rn(by_sc(m[j])))));
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) out[j] = static_cast<int8_t>(max(-127, min(127, __float2int_rn(m[j] / sc))));
        }
        store16(static_cast<int8_t*>(a.m), i0, n, out);
        if (any && (lane & (LANES_B - 1)) == 0) a.ms[blk] = sc;
    }
    // ---- variance store ----
    if constexpr (VB == 4) {
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) mx = fmaxf(mx, root[j]);
        mx = seg_max(mx, 4);
        const float sc = fmaxf(mx / 15.f, 1.e-30f);
        uint32_t vc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float z = fminf(15.f, root[j] / sc);
            const float lo = floorf(z);
            const uint32_t rnd = adam_bits(static_cast<uint32_t>(i0 + j), step, a.key);
            const float uu = static_cast<float>(rnd >> 16) * (1.f / 65536.f);
            vc[j] = static_cast<uint32_t>(fmaxf(static_cast<float>(root[j] > 0.f), fminf(15.f, lo + static_cast<float>(rounds_up(z, lo, uu)))));
        }
        if constexpr (M4) {
            uint8_t out[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) out[j] = static_cast<uint8_t>(mcode[j] | (vc[j] << 4));
            store16(static_cast<uint8_t*>(a.m), i0, n, out);
        } else {
            uint8_t pk[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) pk[j] = static_cast<uint8_t>(vc[2 * j] | (vc[2 * j + 1] << 4));
            const int64_t pn = (n + 1) / 2;
            if (i0 / 2 + 8 <= pn) memcpy(static_cast<uint8_t*>(a.v) + i0 / 2, pk, 8);
            else for (int j = 0; j < 8; ++j) if (i0 / 2 + j < pn) static_cast<uint8_t*>(a.v)[i0 / 2 + j] = pk[j];
        }
        if (any && (lane & 3) == 0) a.vs[i0 / 64] = sc;
    } else if constexpr (VB == 8) {
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) mx = fmaxf(mx, root[j]);
        mx = seg_max(mx, LANES_B);
        const float sc = fmaxf(mx / 255.f, 1.e-30f);
        uint8_t out[16];
        // root <= 255 sc.  A quotient z under 2^-43 only decides "z * z > 0" below, which turns at z near 2^-75; a nonzero
        // root = sqrt(v) is at least 2^-75 (v is a float), so sc is at least 1 there and the remainder is normal
        const SharedDivisor by_sc = shared_divisor(sc);
        float zq[16];
        if (by_sc.safe) {
#pragma unroll
            for (int j = 0; j < 16; ++j) zq[j] = by_sc(root[j]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) zq[j] = root[j] / sc;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float z = fminf(255.f, zq[j]);
            const float lo = floorf(z);
            const uint32_t rnd = adam_bits(static_cast<uint32_t>(i0 + j), step, a.key);
            const float uu = u16_as_float(rnd >> 16) * (1.f / 65536.f);
            const float code = fmaxf(root[j] > 0.f ? 1.f : 0.f, lo + (rounds_up(z, lo, uu) ? 1.f : 0.f));
            out[j] = static_cast<uint8_t>(__float_as_uint(fminf(255.f, code) + 8388608.f));   // integer 0..255 in the low mantissa byte
        }
        store16(static_cast<uint8_t*>(a.v), i0, n, out);
        if (any && (lane & (LANES_B - 1)) == 0) a.vs[blk] = sc;
    } else {
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) mx = fmaxf(mx, v[j]);
        mx = seg_max(mx, LANES_B);
        const float sc = fmaxf(mx / 32768.f, 1.e-35f);
        uint16_t out[16];
        const SharedDivisor by_sc = shared_divisor(sc);     // v <= 32768 sc; a quotient under 2^-43 is zero in FP16
        if (by_sc.safe) {
#pragma unroll
            for (int j = 0; j < 16; ++j) out[j] = __half_as_ushort(__float2half_rn(by_sc(v[j])));
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) out[j] = __half_as_ushort(__float2half_rn(v[j] / sc));
        }
        store16(static_cast<uint16_t*>(a.v), i0, n, out);
        if (any && (lane & (LANES_B - 1)) == 0) a.vs[blk] = sc;
    }
    return amax;
}

// Tensor scale for the next forward, max(amax, 1e-12) * (1 / 2688): block maximum, one atomic per CTA, the last CTA to
// arrive publishes the scale and leaves the two scratch words zeroed.
__device__ __forceinline__ void adam_publish_scale(const AdamArgs& a, float amax) {
    __shared__ float warp_amax[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    amax = seg_max(amax, 32);
    if (lane == 0) warp_amax[warp] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float b = 0.f;
        for (int w = 0; w < 8; ++w) b = fmaxf(b, warp_amax[w]);
        atomicMax(&a.scratch[0], __float_as_uint(b));  // non-negative floats order like their bit patterns
        __threadfence();
        if (atomicAdd(&a.scratch[1], 1u) == gridDim.x - 1) {
            __threadfence();
            const float total = __uint_as_float(atomicExch(&a.scratch[0], 0u));
            a.scale_out[0] = fmaxf(total, 1.e-12f) * (1.f / 2688.f);
            a.scratch[1] = 0u;
        }
    }
}

template <int MASTER, int VB, bool M4, bool NL, int B>
__global__ void __launch_bounds__(256, ADAM_MIN_BLOCKS) adamw_kernel(const AdamArgs a) {
    float c1 = a.c1, c2 = a.c2;
    uint32_t step = a.step;
    if (a.ctrl) { c1 = a.ctrl[0]; c2 = a.ctrl[1]; step = __float_as_uint(a.ctrl[3]); }
    const float amax = adam_chunk<MASTER, VB, M4, NL, B>(a, blockIdx.x, c1, c2, step);
    if (a.scale_out) adam_publish_scale(a, amax);
}

// The update AND the next forward's weight packings in one launch.  Phase 1: a grid of resident CTAs walks the chunks and
// publishes the new tensor scale.  Grid barrier.  Phase 2: the same CTAs walk the 128 x 128 tiles of the updated weight
// (still in L2: a weight is at most a few tens of megabytes) and write both NVFP4 orientations against the new scale,
// byte-identical to quantising the updated weight in the next forward.
// The barrier is an arrival counter in the caller's scratch; the launch asks for no more CTAs than fit the GPU at once
// (cooperative launch), and the wait is bounded: on expiry the status word is raised and phase 2 is skipped.
template <int MASTER, int VB, bool M4, bool NL, int B>
__global__ void __launch_bounds__(256, 4) adamw_prepack_kernel(const AdamArgs a, const PackArgs k) {
    __shared__ PackSmem pack;
    __shared__ int proceed;
    float c1 = a.c1, c2 = a.c2;
    uint32_t step = a.step;
    if (a.ctrl) { c1 = a.ctrl[0]; c2 = a.ctrl[1]; step = __float_as_uint(a.ctrl[3]); }
    const int64_t chunks = (a.n + 4095) / 4096;
    float amax = 0.f;
    for (int64_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x)
        amax = fmaxf(amax, adam_chunk<MASTER, VB, M4, NL, B>(a, chunk, c1, c2, step));
    adam_publish_scale(a, amax);
    // ---- grid barrier: every CTA's master stores and the published scale are visible after it ----
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(k.barrier, 1u);
        const long long t0 = clock64();
        int ok = 1;
        while (*reinterpret_cast<volatile unsigned int*>(k.barrier) < gridDim.x) {
            __nanosleep(200);
            if (clock64() - t0 > 4000000000LL) { ok = 0; break; }
        }
        __threadfence();
        proceed = ok;
        if (!ok && k.status) *k.status = NVFP4_ERR_TIMEOUT;
    }
    __syncthreads();
    if (proceed) {
        const float inv = __fdiv_rn(1.f, __ldcg(a.scale_out));
        const int64_t tiles_c = round128(k.cols) / 128, tiles = (round128(k.rows) / 128) * tiles_c;
        for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) pack_tile<MASTER>(a.p, k, t / tiles_c, t % tiles_c, inv, pack);
    }
    // the last CTA to leave zeroes the barrier word for the next launch
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(k.barrier, 1u) == 2u * gridDim.x - 1u) *k.barrier = 0u;
}

// FP32 moments, FP32 master: tensors below 4096 elements (norm gains, biases).
__global__ void __launch_bounds__(256) adamw_plain_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                          float* __restrict__ m, float* __restrict__ v, int64_t n,
                                                          const float* __restrict__ ctrl, float lr, float decay, float b1,
                                                          float b2, float c1, float c2, float eps, float grad_mul) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (ctrl) { c1 = ctrl[0]; c2 = ctrl[1]; }
    const float one_b1 = 1.f - b1, one_b2 = 1.f - b2, lrc1 = lr * c1;
    float gi = g[i];
    if (grad_mul != 1.f) gi *= grad_mul;
    const float t1 = b1 * m[i], t2 = one_b1 * gi;
    const float mm = t1 + t2;
    const float t3 = b2 * v[i], t4 = (one_b2 * gi) * gi;
    const float vv = t3 + t4;
    p[i] = p[i] * decay - (lrc1 * mm) / (sqrtf(vv) * c2 + eps);
    m[i] = mm;
    v[i] = vv;
}

template <int MASTER, int VB, bool M4, bool NL>
static void launch_block(const AdamArgs& a, int block, unsigned grid, cudaStream_t st) {
    if (block == 512) adamw_kernel<MASTER, VB, M4, NL, 512><<<grid, 256, 0, st>>>(a);
    else if (block == 256) adamw_kernel<MASTER, VB, M4, NL, 256><<<grid, 256, 0, st>>>(a);
    else if (block == 128) adamw_kernel<MASTER, VB, M4, NL, 128><<<grid, 256, 0, st>>>(a);
    else adamw_kernel<MASTER, VB, M4, NL, 64><<<grid, 256, 0, st>>>(a);
}
template <int MASTER>
static bool launch_master(const AdamArgs& a, int vbits, int mbits, int nl, int block, unsigned grid, cudaStream_t st) {
    if (mbits == 8 && vbits == 8) launch_block<MASTER, 8, false, false>(a, block, grid, st);
    else if (mbits == 8 && vbits == 16) launch_block<MASTER, 16, false, false>(a, block, grid, st);
    else if (mbits == 8 && vbits == 4) launch_block<MASTER, 4, false, false>(a, 512, grid, st);
    else if (mbits == 4 && vbits == 4 && nl) launch_block<MASTER, 4, true, true>(a, 512, grid, st);
    else if (mbits == 4 && vbits == 4) launch_block<MASTER, 4, true, false>(a, 512, grid, st);
    else if (mbits == 4 && vbits == 8 && !nl) launch_block<MASTER, 8, true, false>(a, 512, grid, st);
    else return false;
    return true;
}

}  // namespace nvfp4

using namespace nvfp4;

static int fill_adam_args(AdamArgs& a, const char* who, void* p, int master, const void* grad, int grad_kind, int64_t grad_cols,
                          int64_t grad_stride, const float* sa, const float* sb, const float* extra, float grad_mul, void* m, void* v,
                          float* ms, float* vs, int8_t* tail, float* unit, int64_t n, int vbits, int mbits, int state_block, float lr,
                          float decay, float b1, float b2, float c1, float c2, float eps, uint32_t step, uint32_t key,
                          const float* ctrl, float* scale_out, void* scratch) {
    NVFP4_REQUIRE(p && grad && m && ms && vs, NVFP4_ERR_ARG, "%s: null pointer", who);
    NVFP4_REQUIRE(n > 0, NVFP4_ERR_ARG, "%s: empty tensor", who);
    NVFP4_REQUIRE(master == 32 || master == 24 || master == 17 || master == 16 || master == 8, NVFP4_ERR_ARG,
                  "%s: unknown master encoding %d", who, master);
    NVFP4_REQUIRE(state_block == 512 || state_block == 256 || state_block == 128 || state_block == 64, NVFP4_ERR_ARG,
                  "%s: state block must be 64, 128, 256 or 512", who);
    NVFP4_REQUIRE(master != 8 || state_block == 512, NVFP4_ERR_ARG, "%s: FP8 masters use 512-element units", who);
    NVFP4_REQUIRE(grad_kind >= 0 && grad_kind <= 2, NVFP4_ERR_ARG, "%s: unknown gradient kind %d", who, grad_kind);
    NVFP4_REQUIRE(grad_kind != 2 || (sa && sb && grad_cols > 0 && grad_stride >= grad_cols), NVFP4_ERR_ARG,
                  "%s: scaled raw gradients need both scales and a valid stride", who);
    NVFP4_REQUIRE(master != 24 || tail, NVFP4_ERR_ARG, "%s: split masters need the tail tensor", who);
    NVFP4_REQUIRE(master != 8 || unit, NVFP4_ERR_ARG, "%s: FP8 masters need the unit tensor", who);
    NVFP4_REQUIRE(v || (mbits == 4 && vbits == 4), NVFP4_ERR_ARG, "%s: missing variance tensor", who);
    NVFP4_REQUIRE(!scale_out || scratch, NVFP4_ERR_ARG, "%s: the amax reduction needs scratch", who);
    a = AdamArgs{};
    a.p = p; a.grad = grad; a.extra = extra; a.m = m; a.v = v; a.ms = ms; a.vs = vs; a.tail = tail; a.unit = unit;
    a.sa = sa; a.sb = sb; a.ctrl = ctrl; a.scale_out = scale_out;
    a.scratch = scratch ? reinterpret_cast<unsigned int*>(static_cast<char*>(scratch) + SCRATCH_ADAM_OFFSET) : nullptr;
    a.n = n; a.grad_cols = grad_kind == 2 ? grad_cols : 1; a.grad_stride = grad_kind == 2 ? grad_stride : 1; a.grad_kind = grad_kind;
    a.lr = lr; a.decay = decay; a.b1 = b1; a.b2 = b2; a.c1 = c1; a.c2 = c2; a.eps = eps; a.grad_mul = grad_mul;
    a.step = step; a.key = key;
    return NVFP4_OK;
}

extern "C" int nvfp4_adamw_step(void* p, int master, const void* grad, int grad_kind, int64_t grad_cols, int64_t grad_stride,
                                const float* sa, const float* sb, const float* extra, float grad_mul, void* m, void* v,
                                float* ms, float* vs, int8_t* tail, float* unit, int64_t n, int vbits, int mbits,
                                int nonlinear_m, int state_block, float lr, float decay, float b1, float b2, float c1, float c2,
                                float eps, uint32_t step, uint32_t key, const float* ctrl, float* scale_out, void* scratch,
                                nvfp4_stream_t stream) {
    AdamArgs a;
    const int rc = fill_adam_args(a, "nvfp4_adamw_step", p, master, grad, grad_kind, grad_cols, grad_stride, sa, sb, extra, grad_mul, m, v,
                                  ms, vs, tail, unit, n, vbits, mbits, state_block, lr, decay, b1, b2, c1, c2, eps, step, key, ctrl,
                                  scale_out, scratch);
    if (rc != NVFP4_OK) return rc;
    const unsigned grid = static_cast<unsigned>((n + 4095) / 4096);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    bool ok = false;
    switch (master) {
        case 32: ok = launch_master<32>(a, vbits, mbits, nonlinear_m, state_block, grid, st); break;
        case 24: ok = launch_master<24>(a, vbits, mbits, nonlinear_m, state_block, grid, st); break;
        case 17: ok = launch_master<17>(a, vbits, mbits, nonlinear_m, state_block, grid, st); break;
        case 16: ok = launch_master<16>(a, vbits, mbits, nonlinear_m, state_block, grid, st); break;
        default: ok = launch_master<8>(a, vbits, mbits, nonlinear_m, state_block, grid, st); break;
    }
    NVFP4_REQUIRE(ok, NVFP4_ERR_UNSUPPORTED, "nvfp4_adamw_step: no kernel for moments m%d v%d", mbits, vbits);
    return launch_status("nvfp4_adamw_step");
}

// ---- update + next weight packings in one cooperative launch -------------------------------------------------------
namespace nvfp4 {
template <int MASTER, int VB, bool M4, bool NL, int B>
static int launch_prepack(AdamArgs& a, PackArgs& k, cudaStream_t st) {
    auto kernel = adamw_prepack_kernel<MASTER, VB, M4, NL, B>;
    static int resident = 0;   // CTAs that fit the GPU at once (per instantiation; the library serves one GPU model)
    if (!resident) {
        int dev = 0, sms = 0, per_sm = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0) != cudaSuccess || per_sm < 1 || sms < 1) {
            set_error("nvfp4_adamw_step_prepack: cannot size the cooperative grid");
            return NVFP4_ERR_LAUNCH;
        }
        resident = per_sm * sms;
    }
    const int64_t chunks = (a.n + 4095) / 4096;
    const int64_t tiles = (round128(k.rows) / 128) * (round128(k.cols) / 128);
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(std::max(chunks, tiles), resident));
    void* args[] = {&a, &k};
    const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3(grid), dim3(256), args, 0, st);
    if (e != cudaSuccess) {
        set_error("nvfp4_adamw_step_prepack: cooperative launch failed: %s", cudaGetErrorString(e));
        return NVFP4_ERR_LAUNCH;
    }
    return launch_status("nvfp4_adamw_step_prepack");
}
}  // namespace nvfp4

extern "C" int nvfp4_adamw_step_prepack(void* p, int master, const void* grad, int grad_kind, int64_t grad_cols, int64_t grad_stride,
                                        const float* sa, const float* sb, const float* extra, float grad_mul, void* m, void* v,
                                        float* ms, float* vs, int8_t* tail, int64_t rows, int64_t cols, int vbits, int mbits,
                                        int nonlinear_m, int state_block, float lr, float decay, float b1, float b2, float c1,
                                        float c2, float eps, uint32_t step, uint32_t key, const float* ctrl, float* scale_out,
                                        uint8_t* packed, uint8_t* scales, uint8_t* packed_t, uint8_t* scales_t, void* scratch,
                                        int* status, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(rows > 0 && cols > 0 && scale_out && packed && scales && packed_t && scales_t && scratch, NVFP4_ERR_ARG,
                  "nvfp4_adamw_step_prepack: null pointer or empty weight");
    for (const void* q : {static_cast<const void*>(packed), static_cast<const void*>(scales), static_cast<const void*>(packed_t),
                          static_cast<const void*>(scales_t)})
        NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_adamw_step_prepack: outputs must be 16-byte aligned");
    AdamArgs a;
    const int rc = fill_adam_args(a, "nvfp4_adamw_step_prepack", p, master, grad, grad_kind, grad_cols, grad_stride, sa, sb, extra, grad_mul,
                                  m, v, ms, vs, tail, nullptr, rows * cols, vbits, mbits, state_block, lr, decay, b1, b2, c1, c2, eps,
                                  step, key, ctrl, scale_out, scratch);
    if (rc != NVFP4_OK) return rc;
    PackArgs k{packed, scales, packed_t, scales_t, rows, cols,
               reinterpret_cast<unsigned int*>(static_cast<char*>(scratch) + SCRATCH_ADAM_OFFSET + 16), status};
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const bool m8v8 = mbits == 8 && vbits == 8;
    if (master == 17 && m8v8 && state_block == 512) return launch_prepack<17, 8, false, false, 512>(a, k, st);
    if (master == 17 && m8v8 && state_block == 128) return launch_prepack<17, 8, false, false, 128>(a, k, st);
    if (master == 24 && m8v8 && state_block == 512) return launch_prepack<24, 8, false, false, 512>(a, k, st);
    if (master == 32 && mbits == 8 && vbits == 16 && state_block == 512) return launch_prepack<32, 16, false, false, 512>(a, k, st);
    if (master == 17 && mbits == 4 && vbits == 4 && nonlinear_m) return launch_prepack<17, 4, true, true, 512>(a, k, st);
    set_error("nvfp4_adamw_step_prepack: no kernel for master %d with moments m%d v%d and state block %d", master, mbits, vbits, state_block);
    return NVFP4_ERR_UNSUPPORTED;
}

extern "C" int nvfp4_adamw_plain(float* p, const float* grad, float* m, float* v, int64_t n, float grad_mul, float lr, float decay,
                                 float b1, float b2, float c1, float c2, float eps, const float* ctrl, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(p && grad && m && v && n > 0, NVFP4_ERR_ARG, "nvfp4_adamw_plain: null pointer or empty tensor");
    adamw_plain_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        p, grad, m, v, n, ctrl, lr, decay, b1, b2, c1, c2, eps, grad_mul);
    return launch_status("nvfp4_adamw_plain");
}

// FP32 -> FP16 / BF16 head (+ signed residual): the one-off conversion of fresh FP32 weights into master storage.
namespace nvfp4 {
__global__ void split_init_kernel(const float* __restrict__ src, uint16_t* __restrict__ hi, int8_t* __restrict__ tail, int64_t n, int master) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = src[i];
    const uint16_t h = master == 17 ? __half_as_ushort(__float2half_rn(x)) : bf16_bits(x);
    hi[i] = h;
    if (tail) tail[i] = static_cast<int8_t>(signed_tail(x, h));
}
}  // namespace nvfp4

extern "C" int nvfp4_split_init(const float* src, int64_t n, int master, void* hi, int8_t* tail, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(src && hi && n > 0, NVFP4_ERR_ARG, "nvfp4_split_init: null pointer or empty tensor");
    NVFP4_REQUIRE(master == 17 || master == 16 || master == 24, NVFP4_ERR_ARG, "nvfp4_split_init: master must be 17, 16 or 24");
    NVFP4_REQUIRE(master != 24 || tail, NVFP4_ERR_ARG, "nvfp4_split_init: split masters need the tail tensor");
    split_init_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        src, static_cast<uint16_t*>(hi), master == 24 ? tail : nullptr, n, master);
    return launch_status("nvfp4_split_init");
}
