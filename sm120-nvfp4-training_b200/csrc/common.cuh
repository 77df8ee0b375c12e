// Shared device helpers of the NVFP4 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#include "../../include/nvfp4_b200.h"

namespace nvfp4 {

void set_error(const char* fmt, ...);
int launch_status(const char* what);

#define NVFP4_REQUIRE(cond, code, ...)        \
    do {                                      \
        if (!(cond)) {                        \
            ::nvfp4::set_error(__VA_ARGS__);  \
            return (code);                    \
        }                                     \
    } while (0)

// Layout of the caller-provided scratch block (zeroed once, every kernel leaves its part zeroed again):
//   [0, 4112)     amax partials + ticket          (quantize.cu)
//   [4112, 4128)  the four amax results of nvfp4_quantize
//   [4128, 4144)  AdamW: amax bits, ticket        (adamw.cu)
//   [4144, 4148)  AdamW with weight packings: arrival counter of the grid barrier
//   [4148, 4156)  resident quantiser: magnitude maximum, arrival counter of its grid barrier
constexpr int SCRATCH_AMAX_OUT_OFFSET = 4112;
constexpr int SCRATCH_ADAM_OFFSET = 4128;
constexpr int SCRATCH_RESIDENT_OFFSET = 4148;
constexpr int SCRATCH_BYTES = 4160;

__host__ __device__ __forceinline__ int64_t round128(int64_t n) { return (n + 127) / 128 * 128; }

// ---- element loads: every source value enters the quantiser as float(bf16_rne(x)) -------------
__device__ __forceinline__ uint16_t bf16_bits(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float bf16_value(uint16_t h) { return __uint_as_float(static_cast<uint32_t>(h) << 16); }

template <int DT>
__device__ __forceinline__ uint16_t load_as_bf16(const void* p, int64_t i) {
    if constexpr (DT == NVFP4_F32) return bf16_bits(static_cast<const float*>(p)[i]);
    else if constexpr (DT == NVFP4_BF16) return static_cast<const uint16_t*>(p)[i];
    else return bf16_bits(__half2float(static_cast<const __half*>(p)[i]));
}
template <int DT>
__device__ __forceinline__ float load_abs(const void* p, int64_t i) {
    if constexpr (DT == NVFP4_F32) return fabsf(static_cast<const float*>(p)[i]);
    else if constexpr (DT == NVFP4_BF16) return fabsf(bf16_value(static_cast<const uint16_t*>(p)[i]));
    else return fabsf(__half2float(static_cast<const __half*>(p)[i]));
}
template <int DT> struct ElemSize { static constexpr int value = (DT == NVFP4_F32) ? 4 : 2; };

// ---- random sources -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t shr_mul(uint32_t z, uint32_t pow2) {   // z >> k as the high half of z * 2^(32-k)
    uint32_t r;
    asm("mul.hi.u32 %0, %1, %2;" : "=r"(r) : "r"(z), "r"(pow2));
    return r;
}
__device__ __forceinline__ uint32_t hash32_mixed(uint32_t z) {   // finaliser of hash32 on a pre-added input
    z ^= shr_mul(z, 1u << 16); z *= 0x7feb352du; z ^= shr_mul(z, 1u << 17); z *= 0x846ca68bu; z ^= shr_mul(z, 1u << 16);
    return z;
}
__device__ __forceinline__ uint32_t hash32(uint32_t seed, uint32_t index) {
    return hash32_mixed(seed * 0x9e3779b9u + index + 0x85ebca6bu);
}
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}
constexpr uint32_t PHILOX_KEY1 = 0x4e564634u;
__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
        uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
        c = make_uint4(hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0);
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return c;
}
__device__ __forceinline__ float uniform24(uint32_t bits) {
    return static_cast<float>(bits >> 8) * (1.0f / 16777216.0f);
}

// ---- E2M1 stochastic level choice ---------------------------------------------------------------
// x in [0, 6], 24 random bits h24 (u = h24 * 2^-24).  Level spacing is 1/2 below 2, 1 below 4, 2 above, i.e. 2^(e-1)
// with e the exponent of max(x, 1).  With xs = x / spacing (exact), the lower level is floor(xs) steps from zero and
// the round-up probability is frac(xs); "u < p" is h24 < frac(xs) * 2^24, which for the integer h24 is
// h24 < C := ceil(frac(xs) * 2^24).  All of it is one integer sum: with F = ceil(xs * 2^24) = floor(xs) * 2^24 + C,
// F + (2^24 - 1 - h24) has floor(xs) + [h24 < C] in the bits above 24, and adding (e - 127) << 25 puts the level's
// base (0, 2 or 4 steps) there too.  Exact arithmetic on the same real numbers as (x - lo) / (hi - lo) < u, hence
// bit-identical to it.  The caller passes nh = 2^24 - 1 - h24, or a value `bias` short of it.
__device__ __forceinline__ uint32_t sr_code_n(float x, uint32_t nh, uint32_t bias = 0u) {
    const uint32_t ex = __float_as_uint(fmaxf(x, 1.0f)) & 0x7F800000u;            // exponent field 127, 128 or 129
    const float rw24 = __uint_as_float(0x8B800000u - ex);                         // 2^24 / spacing = 2^25, 2^24, 2^23
    const uint32_t f = static_cast<uint32_t>(__float2int_ru(__fmul_rn(x, rw24)));  // < 2^27; the product is exact
    const uint32_t base = (ex << 2) + 0x02000000u + bias;                         // (e - 127) << 25 modulo 2^32
    return (f + nh + base) >> 24;
}
__device__ __forceinline__ uint32_t sr_code(float x, uint32_t h24) { return sr_code_n(x, h24 ^ 0xFFFFFFu); }
__device__ __forceinline__ uint32_t mad_lo(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
// Signed form: the whole 4-bit code (bit 3 = sign, set iff q < 0) of q clamped to [-6, 6].  Same sum as sr_code_n with
// the sign added in as 1 << 27; the integer adds, the shifts and the sign extraction are written as multiply-adds so
// that they run on the FMA pipe, which these kernels leave half idle while the ALU pipe is their limit.  q + 0 turns
// -0 into +0 (round-to-nearest), after which "q < 0" is the sign bit.
__device__ __forceinline__ uint32_t sr_code_signed(float q, uint32_t nh, uint32_t bias = 0u) {
    const float qz = __fadd_rn(q, 0.0f);
    const uint32_t sgn = shr_mul(__float_as_uint(qz), 2u);
    const float x = fminf(fabsf(qz), 6.f);
    const uint32_t ex = __float_as_uint(fmaxf(x, 1.0f)) & 0x7F800000u;
    const float rw24 = __uint_as_float(mad_lo(ex, 0xFFFFFFFFu, 0x8B800000u));
    const uint32_t f = static_cast<uint32_t>(__float2int_ru(__fmul_rn(x, rw24)));
    const uint32_t base = mad_lo(sgn, 0x08000000u, mad_lo(ex, 4u, 0x02000000u + bias));
    return shr_mul(f + nh + base, 256u);
}

// ---- division by a shared divisor -----------------------------------------------------------------
// Many quotients a / b with one divisor b > 0 (a block's scale).  y = RN(1 / b) is taken once per lane; per quotient
// q0 = RN(a y), then twice r = a - b q (exact in an FMA), q = RN(q + r y).  The first correction makes q faithful, and with a
// correctly rounded reciprocal and a faithful quotient the second one returns RN(a / b) (Markstein's theorem on FMA
// division), as long as no remainder is subnormal.  With b in [2^-60, 2^100] (`safe`) that holds for every quotient of at
// least 2^-43; every use below has |a / b| <= 32768 and does not depend on the last bits of a quotient under 2^-43
// (stated at each use).  Outside `safe` the caller divides with `/`.
struct SharedDivisor {
    float b, y;
    bool safe;
    __device__ __forceinline__ float operator()(float a) const {
        float q = __fmul_rn(a, y);
        q = __fmaf_rn(__fmaf_rn(-b, q, a), y, q);
        return __fmaf_rn(__fmaf_rn(-b, q, a), y, q);
    }
};
__device__ __forceinline__ SharedDivisor shared_divisor(float b) {
    return SharedDivisor{b, __frcp_rn(b), b >= 8.673617379884035e-19f && b <= 1.2676506002282294e30f};
}

// ---- scale-factor swizzle (32 x 4 x 4 atom inside 128-row x 4-group blocks) ------------------------
__host__ __device__ __forceinline__ int64_t scale_offset(int64_t row, int64_t group_col, int64_t groups_per_row) {
    return ((row >> 7) * (groups_per_row >> 2) + (group_col >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 +
           (group_col & 3);
}

__device__ __forceinline__ float e4m3_normal_to_float(uint32_t x) {  // positive normal codes only
    return __uint_as_float(((x >> 3) + 120u) << 23 | (x & 7u) << 20);
}
__device__ __forceinline__ float e4m3_to_float(uint32_t x) {   // codes 0x7f / 0xff are NaN
    uint32_t e = (x >> 3) & 15u, m = x & 7u;
    float v = e ? __uint_as_float((e + 120u) << 23 | m << 20) : static_cast<float>(m) * 0.001953125f;
    if ((x & 127u) == 127u) v = __uint_as_float(0x7fc00000u);
    return (x & 128u) ? -v : v;
}
__device__ __forceinline__ float e2m1_to_float(uint32_t c) {
    uint32_t a = c & 7u;
    float v = a < 2u ? static_cast<float>(a) * .5f : __uint_as_float(((a >> 1) + 126u) << 23 | (a & 1u) << 22);
    return (c & 8u) ? -v : v;
}

}  // namespace nvfp4
