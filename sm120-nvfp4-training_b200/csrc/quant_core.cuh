// Group arithmetic of the NVFP4 quantiser, shared by every kernel that emits a packing (tile quantiser, streaming
// quantiser, the optimizer's weight-packing phase).
//
// Numerical contract (bit exact against the CPU oracle): value = float(bf16_rne(x)); optional sign * H16 / 4 butterfly
// over the 16 contraction elements; block scale e4m3_rn(clamp((amax16 / 6) * (1 / pts), 2^-6, 448)); element
// q = v * ((1 / pts) / scale), rounded to e2m1
//   - to nearest by the hardware conversion cvt.rn.satfinite.e2m1x2.f32,
//   - stochastically between adjacent levels with the reference's 24-bit integer hash (clamped to +-6 first), or
//   - stochastically by the hardware conversion cvt.rs.satfinite.e2m1x4.f32 fed with Philox4x32-10 bits.
// All float operations that take part in the contract are written with the _rn intrinsics so the compiler can never
// contract them into FMAs.
#pragma once
#include "common.cuh"

namespace nvfp4 {

// sign * H16 butterfly WITHOUT the final 1/4: that power-of-two factor is folded into the block amax and the element
// multiplier by the caller, which gives the same bits as scaling the 16 values first (a multiplication by 0.25 is
// exact).  The first stage absorbs the signs: a product with +-1 is exact, so fma(b, s_b, a * s_a) rounds once, exactly
// like (a * s_a) + (b * s_b).
__device__ __forceinline__ void hadamard16_unscaled(float (&v)[16], const float (&sg)[16]) {
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const float a = __fmul_rn(v[2 * p], sg[2 * p]);
        const float b = v[2 * p + 1], sb = sg[2 * p + 1];
        v[2 * p] = __fmaf_rn(b, sb, a);
        v[2 * p + 1] = __fmaf_rn(b, -sb, a);
    }
    // stages 2, 4, 8 pair whole (even, odd) couples: two-wide FP32 instructions, each half one IEEE rounding as before
    // (x - y is fma(y, -1, x): the product is exact)
    const float2 minus = make_float2(-1.f, -1.f);
#pragma unroll
    for (int d = 2; d < 16; d <<= 1) {
#pragma unroll
        for (int l = 0; l < 16; l += 2) {
            if (l & d) continue;
            const float2 lo = make_float2(v[l], v[l + 1]), hi = make_float2(v[l ^ d], v[(l ^ d) + 1]);
            const float2 sum = __fadd2_rn(lo, hi), dif = __ffma2_rn(hi, minus, lo);
            v[l] = sum.x; v[l + 1] = sum.y; v[l ^ d] = dif.x; v[(l ^ d) + 1] = dif.y;
        }
    }
}

constexpr int SR_NONE = 0, SR_HASH = 1, SR_PHILOX = 2;
__host__ __device__ constexpr int sr_of_flags(int flags) {
    return (flags & NVFP4_Q_SR_HASH) ? SR_HASH : (flags & NVFP4_Q_SR_PHILOX) ? SR_PHILOX : SR_NONE;
}

// Four floats to four e2m1 codes with the hardware's stochastic rounding.  Result nibbles: d at bits 3:0, c at 7:4, b at
// 11:8, a at 15:12; each value is clamped to +-6 and keeps its sign bit (also on a zero result).  Of the 32 random bits,
// d adds the 16-bit number (byte2 << 8 | byte0) to the 16 fraction bits below its lower level and rounds up on a carry,
// c uses the bit-reversed form of d's number; b uses (byte3 << 8 | byte1), a its bit-reversed form.  (Measured on the
// B200 against the CPU model on 17 million cases; the CPU oracle restates it.)
__device__ __forceinline__ uint32_t cvt_rs_e2m1x4(float a, float b, float c, float d, uint32_t rbits) {
    uint16_t r;
    asm("cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5;" : "=h"(r) : "f"(a), "f"(b), "f"(c), "f"(d), "r"(rbits));
    return r;
}

// Eight floats to one payload word, element 0 in the low nibble, round to nearest even.
__device__ __forceinline__ uint32_t cvt_rn_e2m1x8(float q0, float q1, float q2, float q3, float q4, float q5, float q6, float q7) {
    uint32_t r;
    asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t.reg .b16 h0, h1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n\t"
        "mov.b16 h0, {t0, t1};\n\tmov.b16 h1, {t2, t3};\n\tmov.b32 %0, {h0, h1};\n\t}"
        : "=r"(r) : "f"(q0), "f"(q1), "f"(q2), "f"(q3), "f"(q4), "f"(q5), "f"(q6), "f"(q7));
    return r;
}

// ---- the two divisions of the block-scale arithmetic without the division instruction ------------------------------
// With y the correctly rounded reciprocal of b, q0 = rn(a * y), r = fma(-b, q0, a) (exact) and q = fma(r, y, q0) is the
// correctly rounded quotient a / b as long as nothing underflows.  Checked by enumeration on the host against the IEEE
// division (tests/exact_division.c): a / 6 over every finite non-negative float (identical from 2^-125 up), and a / s
// for every E4M3 mantissa and exponent of s over numerators from 2^-100 to 2^100.  Callers keep to those ranges
// (ScaleMath::fast) and use the division instruction outside them.
__device__ __forceinline__ float div6_exact(float a) {
    const float c = 0.16666667163372039794921875f;   // rn(1 / 6)
    const float q0 = __fmul_rn(a, c);
    return __fmaf_rn(__fmaf_rn(-6.f, q0, a), c, q0);
}
// rn(1 / (1 + m / 8)) for the eight E4M3 mantissas
static __constant__ uint32_t E4M3_RCP_MANTISSA[8] = {0x3f800000u, 0x3f638e39u, 0x3f4ccccdu, 0x3f3a2e8cu,
                                              0x3f2aaaabu, 0x3f1d89d9u, 0x3f124925u, 0x3f088889u};
// a / value(e8) for a positive normal E4M3 code e8
__device__ __forceinline__ float div_e4m3_exact(float a, uint32_t e8) {
    const float s = e4m3_normal_to_float(e8);
    const float y = __uint_as_float(E4M3_RCP_MANTISSA[e8 & 7u] + ((7u - (e8 >> 3)) << 23));
    const float q0 = __fmul_rn(a, y);
    return __fmaf_rn(__fmaf_rn(-s, q0, a), y, q0);
}

struct ScaleMath {
    float inv;    // 1 / tensor scale
    bool fast;    // inv inside [2^-100, 2^100]: the division-free forms give the IEEE quotients
};
__device__ __forceinline__ ScaleMath scale_math(float pts) {
    ScaleMath m;
    m.inv = __fdiv_rn(1.f, pts);
    m.fast = m.inv >= 7.888609052210118e-31f && m.inv <= 1.2676506002282294e30f;
    return m;
}

// Encodes 16 values (times `fold` = 0.25 when they come from hadamard16_unscaled, else 1).
// idx0 = flat index of element 0 in the packing's padded coordinates (a multiple of 16).
__device__ __forceinline__ uint2 swap_nibbles(uint2 p) {   // Comfy order: even element in the high nibble
    p.x = ((p.x & 0x0f0f0f0fu) << 4) | ((p.x >> 4) & 0x0f0f0f0fu);
    p.y = ((p.y & 0x0f0f0f0fu) << 4) | ((p.y >> 4) & 0x0f0f0f0fu);
    return p;
}

// FAST: the caller has checked ScaleMath::fast for the whole launch (a branch per group costs more than it saves).
// hash_idx0 = low 32 bits of the flat index of element 0, group = that index / 16 (the Philox counter).
template <int SR, bool FAST>
__device__ __forceinline__ uint2 encode16(const float (&v)[16], bool fold, float inv, uint32_t seed, uint32_t hash_idx0,
                                          uint64_t group, uint32_t& scale_byte) {
    float a = 0.f;
#pragma unroll
    for (int l = 0; l < 16; ++l) a = fmaxf(a, fabsf(v[l]));
    if (fold) a = __fmul_rn(a, 0.25f);
    // a / 6: below 2^-125 the two forms may differ in the last bit, but there the product with inv <= 2^100 is far under
    // the 2^-6 floor, so the scale byte is the same
    const float sixth = FAST ? div6_exact(a) : __fdiv_rn(a, 6.f);
    const float enc = fminf(fmaxf(__fmul_rn(sixth, inv), 0.015625f), 448.f);
    const uint32_t e8 = __nv_cvt_float_to_fp8(enc, __NV_SATFINITE, __NV_E4M3);
    scale_byte = e8;
    float mul = FAST ? div_e4m3_exact(inv, e8) : __fdiv_rn(inv, e4m3_normal_to_float(e8));
    if (fold) mul = __fmul_rn(mul, 0.25f);
    float q[16];   // v * mul, two per instruction
    const float2 mul2 = make_float2(mul, mul);
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const float2 t = __fmul2_rn(make_float2(v[2 * p], v[2 * p + 1]), mul2);
        q[2 * p] = t.x; q[2 * p + 1] = t.y;
    }
    uint32_t lo = 0, hi = 0;
    if constexpr (SR == SR_NONE) {
        // cvt.rn.satfinite clamps to +-6 by itself; the first source operand lands in the high nibble.  Eight values
        // become one word: four conversions, whose bytes are packed by register moves.
        lo = cvt_rn_e2m1x8(q[0], q[1], q[2], q[3], q[4], q[5], q[6], q[7]);
        hi = cvt_rn_e2m1x8(q[8], q[9], q[10], q[11], q[12], q[13], q[14], q[15]);
    } else if constexpr (SR == SR_PHILOX) {
        // one Philox block per group: word j rounds elements 4j .. 4j+3
        const uint4 r = philox4x32_10(make_uint4(static_cast<uint32_t>(group), static_cast<uint32_t>(group >> 32), 0u, 0u), seed, PHILOX_KEY1);
        const uint32_t d0 = cvt_rs_e2m1x4(q[3], q[2], q[1], q[0], r.x), d1 = cvt_rs_e2m1x4(q[7], q[6], q[5], q[4], r.y);
        const uint32_t d2 = cvt_rs_e2m1x4(q[11], q[10], q[9], q[8], r.z), d3 = cvt_rs_e2m1x4(q[15], q[14], q[13], q[12], r.w);
        lo = __byte_perm(d0, d1, 0x5410);
        hi = __byte_perm(d2, d3, 0x5410);
    } else {
        uint32_t codes[16];
        const uint32_t hbase = seed * 0x9e3779b9u + hash_idx0 + 0x85ebca6bu;
#pragma unroll
        for (int l = 0; l < 16; ++l) {
            // complement of the 24 random bits (the level choice adds it)
            const uint32_t nh = shr_mul(~hash32_mixed(hbase + l), 1u << 24);
            codes[l] = sr_code_signed(q[l], nh);   // sign bit set iff q < 0 (so -0 encodes as +0)
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            lo |= (codes[2 * b] | (codes[2 * b + 1] << 4)) << (8 * b);
            hi |= (codes[8 + 2 * b] | (codes[8 + 2 * b + 1] << 4)) << (8 * b);
        }
    }
    return make_uint2(lo, hi);
}

// Tensor scale of one orientation: read from `pts`, or, when a producer kernel left the tensor's amax on the device,
// computed from it with the expression of the amax kernel, (factor * max(amax, 1e-12)) * (1 / 2688) with factor 4 under
// the Hadamard transform, and written to `pts` by the first thread of the grid (the GEMM reads it from there).
__device__ __forceinline__ float tensor_scale(const float* amax, float* pts, bool rht, bool writer) {
    if (!amax) return __ldg(pts);
    const float a = fmaxf(bf16_value(bf16_bits(__ldg(amax))), 1.e-12f);
    const float v = __fmul_rn(__fmul_rn(rht ? 4.f : 1.f, a), 1.f / (6.f * 448.f));
    if (writer) *pts = v;
    return v;
}

struct Orient {
    uint8_t* packed;
    uint8_t* scales;
    float* pts;
    int64_t kp;  // padded contraction extent of this packing
    uint32_t seed;
    int flags;
};

}  // namespace nvfp4
