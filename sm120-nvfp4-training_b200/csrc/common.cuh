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
constexpr int SCRATCH_AMAX_OUT_OFFSET = 4112;
constexpr int SCRATCH_ADAM_OFFSET = 4128;
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
__device__ __forceinline__ uint32_t hash32(uint32_t seed, uint32_t index) {
    uint32_t z = seed * 0x9e3779b9u + index + 0x85ebca6bu;
    z ^= z >> 16; z *= 0x7feb352du; z ^= z >> 15; z *= 0x846ca68bu; z ^= z >> 16;
    return z;
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
__device__ __forceinline__ uint32_t sr_magnitude(float x, float u) {
    // x in [0, 6].  Level spacing is 1/2 below 2, 1 below 4, 2 above; t counts whole steps from zero of
    // that spacing, lo = t * spacing is the level at or below x.  (x - lo) / spacing is written as a product:
    // the spacing is a power of two, so both forms round to the same float.  x == 6 gives lo = 4, p = 1 > u.
    const bool s2 = x < 2.f, s4 = x < 4.f;
    const float rw = s2 ? 2.f : (s4 ? 1.f : .5f);
    const float w = s2 ? .5f : (s4 ? 1.f : 2.f);
    const float t = s4 ? floorf(__fmul_rn(x, rw)) : 2.f;
    const float lo = __fmul_rn(t, w);
    const uint32_t code = static_cast<uint32_t>(t) + (s2 ? 0u : (s4 ? 2u : 4u));
    return code + static_cast<uint32_t>(u < __fmul_rn(__fsub_rn(x, lo), rw));
}

// ---- scale-factor swizzle (32 x 4 x 4 atom inside 128-row x 4-group blocks) ------------------------
__host__ __device__ __forceinline__ int64_t scale_offset(int64_t row, int64_t group_col, int64_t groups_per_row) {
    return ((row >> 7) * (groups_per_row >> 2) + (group_col >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 +
           (group_col & 3);
}

__device__ __forceinline__ float e4m3_normal_to_float(uint32_t x) {  // positive normal codes only
    return __uint_as_float(((x >> 3) + 120u) << 23 | (x & 7u) << 20);
}
__device__ __forceinline__ float e4m3_to_float(uint32_t x) {
    uint32_t e = (x >> 3) & 15u, m = x & 7u;
    float v = e ? __uint_as_float((e + 120u) << 23 | m << 20) : static_cast<float>(m) * 0.001953125f;
    return (x & 128u) ? -v : v;
}
__device__ __forceinline__ float e2m1_to_float(uint32_t c) {
    uint32_t a = c & 7u;
    float v = a < 2u ? static_cast<float>(a) * .5f : __uint_as_float(((a >> 1) + 126u) << 23 | (a & 1u) << 22);
    return (c & 8u) ? -v : v;
}

}  // namespace nvfp4
