// nvcc-flags: --fmad=false
// Kernels behind PackedNVFP4Linear: frozen NVFP4 checkpoints in "Comfy" order (even element in the HIGH nibble,
// E4M3 block scales in the 128 x 4 swizzle, one FP32 tensor scale) used as LoRA bases.
//
// Numerical contract, shared with the CPU oracle (the arithmetic of the reference's
// src/precision_lora/_packed_cuda.py:14-55,64-103,117-163, restated; compiled without FMA contraction like there):
//   dequantise   scale = bf16(g * e4m3(s)); value = bf16(e2m1(code) * scale)
//   quantise     v = bf16 input, optionally rotated by sign * H128 / sqrt(128) over each aligned run of 128 columns
//                (butterfly over index bits 0..6 in that order, difference = lower-index element minus higher);
//                g = max(amax(v) / 2688, 1e-30); block scale sc = e4m3_rne(max16 / (6 g)) in software with 0 and 448
//                clamps; q = v / (e4m3(sc) g) (0 when that product is 0), rounded to E2M1 by the hardware RNE
//                conversion or stochastically: round up iff (mix32(index ^ seed) >> 8) 2^-24 < (|q| - lo) / (hi - lo)
//   transpose + rotate + requantise   the packed weight is decoded as above, multiplied by the signs along the output-
//                feature axis, rotated along that axis and requantised (RNE) against a separate tensor scale, giving
//                the operand of the input-gradient GEMM without ever materialising a dense weight.
// Differences from the reference are in organisation only: the rotation is fused into both the amax and the quantise
// pass (no FP32 workspace), every thread moves 16-byte vectors, scale bytes are written as whole 32-bit words, and
// the transpose kernel works on 128 x 128 tiles staged as BF16 in shared memory.
#include "common.cuh"

#include <algorithm>

namespace nvfp4 {

constexpr float H128_NORM = 0.08838834764831845f;

// ---- scalar pieces ------------------------------------------------------------------------------
__device__ __forceinline__ uint16_t bf16_rne_bits(float x) {   // integer RNE (finite inputs)
    const uint32_t u = __float_as_uint(x);
    return static_cast<uint16_t>((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
__device__ __forceinline__ float bf16_round(float x) { return bf16_value(bf16_rne_bits(x)); }

__device__ __forceinline__ uint32_t e4m3_encode_soft(float v) {   // non-negative input, RNE, saturating at 448
    if (v <= 0.0f) return 0u;
    if (v >= 448.0f) return 126u;
    int e = static_cast<int>((__float_as_uint(v) >> 23) & 255u) - 127;
    if (e < -6) return static_cast<uint32_t>(__float2int_rn(v * 512.0f));
    int m = __float2int_rn(v * __uint_as_float(static_cast<uint32_t>(130 - e) << 23)) - 8;
    if (m == 8) { ++e; m = 0; }
    return static_cast<uint32_t>(((e + 7) << 3) | m);
}

__device__ __forceinline__ uint32_t e2m1_pair_hi_first(float even, float odd) {   // one byte: even element high
    return static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(make_float2(odd, even), __NV_E2M1, cudaRoundNearest));
}
__device__ __forceinline__ uint32_t e2m1_stochastic(float q, uint32_t bits) {
    const float a = fabsf(q);
    const uint32_t mag = a >= 6.0f ? 7u : sr_code(a, bits >> 8);
    return mag | (signbit(q) ? 8u : 0u);
}

// sign * H128 / sqrt(128) over 128 values held 8 per lane by 16 consecutive lanes (element j = lane16 * 8 + e)
__device__ __forceinline__ void rotate128(float (&v)[8], int lane16) {
#pragma unroll
    for (int d = 1; d < 8; d <<= 1)
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (!(e & d)) { const float a = v[e], b = v[e | d]; v[e] = a + b; v[e | d] = a - b; }
#pragma unroll
    for (int m = 1; m < 16; m <<= 1)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, v[e], m);
            v[e] = (lane16 & m) ? other - v[e] : v[e] + other;
        }
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] *= H128_NORM;
}

__device__ __forceinline__ void load8(const uint16_t* p, float (&v)[8]) {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __uint_as_float(u[i] << 16); v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
}

// ---- amax of the (optionally rotated) BF16 input ---------------------------------------------
template <bool ROT>
__global__ void __launch_bounds__(256) comfy_amax_kernel(const uint16_t* __restrict__ x, const float* __restrict__ signs,
                                                         int64_t segments, uint32_t* __restrict__ amax_bits) {
    const int lane16 = threadIdx.x & 15;
    float sg[8];
    if constexpr (ROT) {
#pragma unroll
        for (int e = 0; e < 8; ++e) sg[e] = signs[lane16 * 8 + e];
    }
    float best = 0.f;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 16;
    // whole warps stay in the loop together (the rotation shuffles across 16 lanes)
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * 16 + (threadIdx.x >> 5) * 2; base < segments; base += stride) {
        const int64_t seg = base + ((threadIdx.x >> 4) & 1);
        float v[8];
        if (seg < segments) load8(x + seg * 128 + lane16 * 8, v);
        else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = 0.f;
        }
        if constexpr (ROT) {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] *= sg[e];
            rotate128(v, lane16);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) best = fmaxf(best, fabsf(v[e]));
    }
#pragma unroll
    for (int m = 16; m; m >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, m));
    __shared__ float warp_best[8];
    if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < 8; ++w) best = fmaxf(best, warp_best[w]);
        atomicMax(amax_bits, __float_as_uint(best));   // non-negative floats order like their bit patterns
    }
}

__global__ void comfy_finish_scale_kernel(const float* amax, float* scale) { scale[0] = fmaxf(amax[0] / 2688.0f, 1.0e-30f); }

// ---- quantiser -------------------------------------------------------------------------------
// x [rows][cols] BF16 contiguous, cols % 128 == 0.  Payload rows [0, rows16) are written (rows beyond `rows` as zeros),
// scale rows [0, rows128) likewise, so the caller needs no memset.
template <bool ROT, bool SR>
__global__ void __launch_bounds__(256) comfy_quant_kernel(const uint16_t* __restrict__ x, const float* __restrict__ signs,
                                                          const float* __restrict__ amax, uint8_t* __restrict__ q,
                                                          uint8_t* __restrict__ s, float* __restrict__ g_out, int64_t rows,
                                                          int64_t rows16, int64_t rows128, int64_t cols, uint32_t seed,
                                                          const uint32_t* __restrict__ counter) {
    const int lane16 = threadIdx.x & 15;
    const int64_t per_row = cols >> 7, segments = rows128 * per_row;
    const float g = fmaxf(amax[0] / 2688.0f, 1.0e-30f);
    const float six_g = 6.0f * g;
    if constexpr (SR) { if (counter) seed += counter[0]; }
    if (blockIdx.x == 0 && threadIdx.x == 0) g_out[0] = g;
    float sg[8];
    if constexpr (ROT) {
#pragma unroll
        for (int e = 0; e < 8; ++e) sg[e] = signs[lane16 * 8 + e];
    }
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 16;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * 16 + (threadIdx.x >> 5) * 2; base < segments; base += stride) {
        const int64_t seg = base + ((threadIdx.x >> 4) & 1);
        const bool live = seg < segments;
        const int64_t r = live ? seg / per_row : 0;
        const int64_t c = live ? (seg - r * per_row) * 128 + lane16 * 8 : 0;
        float v[8];
        if (live && r < rows) load8(x + r * cols + c, v);
        else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = 0.f;
        }
        if constexpr (ROT) {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] *= sg[e];
            rotate128(v, lane16);
        }
        float a = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) a = fmaxf(a, fabsf(v[e]));
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
        const uint32_t sc = e4m3_encode_soft(a / six_g);
        const float total = e4m3_to_float(sc) * g;
        float n[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) n[e] = total == 0.f ? 0.f : v[e] / total;
        uint32_t word = 0;
        if constexpr (SR) {
            const uint32_t index = static_cast<uint32_t>(r * cols + c);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t code = e2m1_stochastic(n[e], mix32((index + e) ^ seed));
                word |= code << (8 * (e >> 1) + ((e & 1) ? 0 : 4));
            }
        } else {
#pragma unroll
            for (int b = 0; b < 4; ++b) word |= e2m1_pair_hi_first(n[2 * b], n[2 * b + 1]) << (8 * b);
        }
        // four block scales of 64 columns form one aligned word of the swizzled layout
        uint32_t packed_scales = sc;
        packed_scales |= __shfl_down_sync(0xffffffffu, sc, 2) << 8;
        packed_scales |= __shfl_down_sync(0xffffffffu, sc, 4) << 16;
        packed_scales |= __shfl_down_sync(0xffffffffu, sc, 6) << 24;
        if (live) {
            if (r < rows16) *reinterpret_cast<uint32_t*>(q + ((r * cols + c) >> 1)) = word;
            if ((lane16 & 7) == 0)
                *reinterpret_cast<uint32_t*>(s + scale_offset(r, c >> 4, cols >> 4)) = packed_scales;
        }
    }
}

// ---- dequantiser ------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) comfy_dequant_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ s,
                                                            const float* __restrict__ g, uint16_t* __restrict__ y, int64_t n,
                                                            int64_t k) {
    const int64_t groups = k >> 4, total = n * groups;
    const float tensor_scale = g[0];
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / groups, b = i - r * groups;
        // widths that are not multiples of 64 still own whole 512-byte scale blocks
        const float scale = bf16_round(tensor_scale * e4m3_to_float(s[scale_offset(r, b, (groups + 3) & ~int64_t(3))]));
        const uint2 p = *reinterpret_cast<const uint2*>(q + i * 8);
        const uint32_t w[2] = {p.x, p.y};
        uint32_t out[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t byte = (w[j >> 2] >> (8 * (j & 3))) & 0xffu;
            const uint32_t even = bf16_rne_bits(e2m1_to_float(byte >> 4) * scale);
            const uint32_t odd = bf16_rne_bits(e2m1_to_float(byte & 15u) * scale);
            out[j] = even | (odd << 16);
        }
        uint4* dst = reinterpret_cast<uint4*>(y + i * 16);
        dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
        dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
    }
}

// ---- packed [n][k] -> packed, rotated [k][n] ---------------------------------------------------
constexpr int TP = 132;   // BF16 elements per shared-memory row: 264 bytes keeps 8-byte row reads aligned
template <bool AMAX_ONLY>
__global__ void __launch_bounds__(256) comfy_transpose_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ scales,
                                                              const float* __restrict__ global, const float* __restrict__ signs,
                                                              const float* __restrict__ backward_global,
                                                              uint8_t* __restrict__ qt, uint8_t* __restrict__ st, int64_t n,
                                                              int64_t k, uint32_t* __restrict__ amax_bits) {
    __shared__ __align__(16) uint16_t tile[128 * TP];   // [k within tile][n within tile], sign already applied
    const int tid = threadIdx.x;
    const int64_t k0 = static_cast<int64_t>(blockIdx.x) * 128, n0 = static_cast<int64_t>(blockIdx.y) * 128;
    {
        // phase 1: thread = (row r, 64-column half); two 16-byte payload loads and one word of four block scales
        const int r = tid >> 1, half = tid & 1;
        const int64_t row = n0 + r, col = k0 + half * 64;
        const uint4* src = reinterpret_cast<const uint4*>(q + ((row * k + col) >> 1));
        const uint4 p0 = src[0], p1 = src[1];
        const uint32_t sw = *reinterpret_cast<const uint32_t*>(scales + scale_offset(row, col >> 4, k >> 4));
        const uint32_t flip = signs[r] < 0.f ? 0x8000u : 0u;   // signs are +-1: the product is a sign flip
        const float tensor_scale = global[0];
        const uint32_t w[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        uint16_t* column = tile + half * 64 * TP + r;
#pragma unroll
        for (int grp = 0; grp < 4; ++grp) {
            const float sc = bf16_round(tensor_scale * e4m3_to_float((sw >> (8 * grp)) & 0xffu));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t byte = (w[grp * 2 + (j >> 2)] >> (8 * (j & 3))) & 0xffu;
                const int kk = grp * 16 + j * 2;
                // both codes of the byte in one conversion (exact in FP16); .x is the low nibble, the odd element here
                const __half2_raw pair = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>(byte), __NV_E2M1);
                column[kk * TP] = static_cast<uint16_t>(bf16_rne_bits(__half2float(__ushort_as_half(pair.y)) * sc) ^ flip);
                column[(kk + 1) * TP] = static_cast<uint16_t>(bf16_rne_bits(__half2float(__ushort_as_half(pair.x)) * sc) ^ flip);
            }
        }
    }
    __syncthreads();
    // phase 2: a warp owns 16 of the tile's k rows; lane = 4 consecutive n, so one row is one 128-point transform
    const int warp = tid >> 5, lane = tid & 31;
    float g = 0.f, six_g = 0.f;
    if constexpr (!AMAX_ONLY) { g = backward_global[0]; six_g = 6.0f * g; }
    float best = 0.f;
    for (int kr = warp; kr < 128; kr += 8) {
        const uint2 raw = *reinterpret_cast<const uint2*>(tile + kr * TP + lane * 4);
        float v[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                      __uint_as_float(raw.y & 0xffff0000u)};
        {
            const float a = v[0], b = v[1], c = v[2], d = v[3];
            const float s0 = a + b, d0 = a - b, s1 = c + d, d1 = c - d;
            v[0] = s0 + s1; v[1] = d0 + d1; v[2] = s0 - s1; v[3] = d0 - d1;
        }
#pragma unroll
        for (int m = 1; m < 32; m <<= 1)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float other = __shfl_xor_sync(0xffffffffu, v[e], m);
                v[e] = (lane & m) ? other - v[e] : v[e] + other;
            }
        float a = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) { v[e] *= H128_NORM; a = fmaxf(a, fabsf(v[e])); }
        if constexpr (AMAX_ONLY) {
            best = fmaxf(best, a);
        } else {
            a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
            a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
            const uint32_t sc = e4m3_encode_soft(a / six_g);
            const float total = e4m3_to_float(sc) * g;
            // four quotients by one divisor: the shared-reciprocal form returns the IEEE quotient for every quotient that can
            // round to a non-zero code (common.cuh); totals outside its range take `/`
            float nq[4];
            const SharedDivisor by_total = shared_divisor(total);
            if (by_total.safe) {
#pragma unroll
                for (int e = 0; e < 4; ++e) nq[e] = by_total(v[e]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) nq[e] = total == 0.f ? 0.f : v[e] / total;
            }
            const uint32_t two = e2m1_pair_hi_first(nq[0], nq[1]) | (e2m1_pair_hi_first(nq[2], nq[3]) << 8);
            const uint32_t next = __shfl_down_sync(0xffffffffu, two, 1);
            uint32_t packed_scales = sc;
            packed_scales |= __shfl_down_sync(0xffffffffu, sc, 4) << 8;
            packed_scales |= __shfl_down_sync(0xffffffffu, sc, 8) << 16;
            packed_scales |= __shfl_down_sync(0xffffffffu, sc, 12) << 24;
            const int64_t out_row = k0 + kr, out_col = n0 + lane * 4;
            if (!(lane & 1)) *reinterpret_cast<uint32_t*>(qt + ((out_row * n + out_col) >> 1)) = two | (next << 16);
            if (!(lane & 15)) *reinterpret_cast<uint32_t*>(st + scale_offset(out_row, out_col >> 4, n >> 4)) = packed_scales;
        }
    }
    if constexpr (AMAX_ONLY) {
#pragma unroll
        for (int m = 16; m; m >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, m));
        if (lane == 0) atomicMax(amax_bits, __float_as_uint(best));
    }
}

// ---- rotary embedding by 2 x 2 matrices --------------------------------------------------------
// x, y [rows][heads][dim] BF16; rot [rows][pairs][2][2] BF16.  For d < 2 * pairs the pair (x[p], x[p + pairs]) is
// multiplied by rot (by its transpose when backward); the remaining features are copied.
__global__ void __launch_bounds__(256) comfy_rope_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ rot,
                                                         uint16_t* __restrict__ y, int64_t rows, int heads, int dim, int pairs,
                                                         int backward) {
    const int64_t total = rows * heads * dim;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int d = static_cast<int>(i % dim);
        if (d >= pairs * 2) { y[i] = x[i]; continue; }
        const int64_t base = i - d, row = i / (static_cast<int64_t>(heads) * dim);
        const int p = d % pairs;
        const uint2 m = *reinterpret_cast<const uint2*>(rot + (row * pairs + p) * 4);
        const float a = bf16_value(x[base + p]), b = bf16_value(x[base + p + pairs]);
        const float r00 = __uint_as_float(m.x << 16), r01 = __uint_as_float(m.x & 0xffff0000u);
        const float r10 = __uint_as_float(m.y << 16), r11 = __uint_as_float(m.y & 0xffff0000u);
        const float v = backward ? (d < pairs ? a * r00 + b * r10 : a * r01 + b * r11)
                                 : (d < pairs ? a * r00 + b * r01 : a * r10 + b * r11);
        y[i] = bf16_rne_bits(v);
    }
}

static int grid_for(int64_t work_items, int per_block) {
    int sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t want = (work_items + per_block - 1) / per_block;
    return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, static_cast<int64_t>(sms) * 8)));
}

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_comfy_quantize(const void* x, int64_t rows, int64_t cols, const float* signs128, int sr, uint32_t seed,
                                    const int32_t* counter, uint8_t* packed, uint8_t* scales, float* tensor_scale,
                                    float* amax_scratch, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(x && packed && scales && tensor_scale && amax_scratch, NVFP4_ERR_ARG, "nvfp4_comfy_quantize: null pointer");
    NVFP4_REQUIRE(rows > 0 && cols > 0 && cols % 128 == 0, NVFP4_ERR_ARG,
                  "nvfp4_comfy_quantize: rows must be positive and cols a positive multiple of 128 (got %lld x %lld)",
                  static_cast<long long>(rows), static_cast<long long>(cols));
    NVFP4_REQUIRE(aligned(x, 16) && aligned(packed, 4) && aligned(scales, 4), NVFP4_ERR_ALIGN,
                  "nvfp4_comfy_quantize: x needs 16-byte, outputs 4-byte alignment");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int64_t rows16 = (rows + 15) / 16 * 16, rows128 = round128(rows);
    const uint16_t* src = static_cast<const uint16_t*>(x);
    uint32_t* amax_bits = reinterpret_cast<uint32_t*>(amax_scratch);
    if (cudaMemsetAsync(amax_scratch, 0, sizeof(float), st) != cudaSuccess) return launch_status("nvfp4_comfy_quantize memset");
    const int64_t live_segments = rows * (cols / 128), all_segments = rows128 * (cols / 128);
    const int g1 = grid_for(live_segments, 16), g2 = grid_for(all_segments, 16);
    const uint32_t* ctr = reinterpret_cast<const uint32_t*>(counter);
    if (signs128) {
        comfy_amax_kernel<true><<<g1, 256, 0, st>>>(src, signs128, live_segments, amax_bits);
        if (sr) comfy_quant_kernel<true, true><<<g2, 256, 0, st>>>(src, signs128, amax_scratch, packed, scales, tensor_scale, rows, rows16, rows128, cols, seed, ctr);
        else comfy_quant_kernel<true, false><<<g2, 256, 0, st>>>(src, signs128, amax_scratch, packed, scales, tensor_scale, rows, rows16, rows128, cols, seed, ctr);
    } else {
        comfy_amax_kernel<false><<<g1, 256, 0, st>>>(src, nullptr, live_segments, amax_bits);
        if (sr) comfy_quant_kernel<false, true><<<g2, 256, 0, st>>>(src, nullptr, amax_scratch, packed, scales, tensor_scale, rows, rows16, rows128, cols, seed, ctr);
        else comfy_quant_kernel<false, false><<<g2, 256, 0, st>>>(src, nullptr, amax_scratch, packed, scales, tensor_scale, rows, rows16, rows128, cols, seed, ctr);
    }
    return launch_status("nvfp4_comfy_quantize");
}

extern "C" int nvfp4_comfy_dequantize(const uint8_t* packed, const uint8_t* scales, const float* tensor_scale, void* out,
                                      int64_t n, int64_t k, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(packed && scales && tensor_scale && out, NVFP4_ERR_ARG, "nvfp4_comfy_dequantize: null pointer");
    NVFP4_REQUIRE(n > 0 && k > 0 && k % 16 == 0, NVFP4_ERR_ARG, "nvfp4_comfy_dequantize: k must be a positive multiple of 16");
    NVFP4_REQUIRE(aligned(packed, 8) && aligned(out, 16), NVFP4_ERR_ALIGN, "nvfp4_comfy_dequantize: misaligned buffers");
    comfy_dequant_kernel<<<grid_for(n * (k / 16), 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        packed, scales, tensor_scale, static_cast<uint16_t*>(out), n, k);
    return launch_status("nvfp4_comfy_dequantize");
}

static int transpose_args(const char* who, const void* q, const void* s, const void* g, const void* signs, int64_t n, int64_t k) {
    NVFP4_REQUIRE(q && s && g && signs, NVFP4_ERR_ARG, "%s: null pointer", who);
    NVFP4_REQUIRE(n > 0 && k > 0 && n % 128 == 0 && k % 128 == 0 && n / 128 <= 65535, NVFP4_ERR_ARG,
                  "%s: n and k must be positive multiples of 128 (got %lld x %lld)", who, static_cast<long long>(n),
                  static_cast<long long>(k));
    NVFP4_REQUIRE(aligned(q, 16) && aligned(s, 4), NVFP4_ERR_ALIGN, "%s: payload needs 16-byte, scales 4-byte alignment", who);
    return NVFP4_OK;
}

extern "C" int nvfp4_comfy_backward_scale(const uint8_t* packed, const uint8_t* scales, const float* tensor_scale,
                                          const float* signs128, int64_t n, int64_t k, float* amax_scratch,
                                          float* backward_scale, nvfp4_stream_t stream) {
    if (int rc = transpose_args("nvfp4_comfy_backward_scale", packed, scales, tensor_scale, signs128, n, k)) return rc;
    NVFP4_REQUIRE(amax_scratch && backward_scale, NVFP4_ERR_ARG, "nvfp4_comfy_backward_scale: null output");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(amax_scratch, 0, sizeof(float), st) != cudaSuccess) return launch_status("nvfp4_comfy_backward_scale memset");
    comfy_transpose_kernel<true><<<dim3(static_cast<unsigned>(k / 128), static_cast<unsigned>(n / 128)), 256, 0, st>>>(
        packed, scales, tensor_scale, signs128, nullptr, nullptr, nullptr, n, k, reinterpret_cast<uint32_t*>(amax_scratch));
    comfy_finish_scale_kernel<<<1, 1, 0, st>>>(amax_scratch, backward_scale);
    return launch_status("nvfp4_comfy_backward_scale");
}

extern "C" int nvfp4_comfy_transpose_requant(const uint8_t* packed, const uint8_t* scales, const float* tensor_scale,
                                             const float* signs128, const float* backward_scale, uint8_t* packed_t,
                                             uint8_t* scales_t, int64_t n, int64_t k, nvfp4_stream_t stream) {
    if (int rc = transpose_args("nvfp4_comfy_transpose_requant", packed, scales, tensor_scale, signs128, n, k)) return rc;
    NVFP4_REQUIRE(backward_scale && packed_t && scales_t && aligned(packed_t, 4) && aligned(scales_t, 4), NVFP4_ERR_ARG,
                  "nvfp4_comfy_transpose_requant: null or misaligned output");
    comfy_transpose_kernel<false><<<dim3(static_cast<unsigned>(k / 128), static_cast<unsigned>(n / 128)), 256, 0,
                                    reinterpret_cast<cudaStream_t>(stream)>>>(packed, scales, tensor_scale, signs128, backward_scale,
                                                                              packed_t, scales_t, n, k, nullptr);
    return launch_status("nvfp4_comfy_transpose_requant");
}

extern "C" int nvfp4_comfy_finish_scale(const float* amax, float* scale, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(amax && scale, NVFP4_ERR_ARG, "nvfp4_comfy_finish_scale: null pointer");
    comfy_finish_scale_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(amax, scale);
    return launch_status("nvfp4_comfy_finish_scale");
}

extern "C" int nvfp4_comfy_rope(const void* x, const void* rotation, void* out, int64_t rows, int heads, int dim, int pairs,
                                int backward, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(x && rotation && out, NVFP4_ERR_ARG, "nvfp4_comfy_rope: null pointer");
    NVFP4_REQUIRE(rows > 0 && heads > 0 && dim > 0 && pairs >= 0 && pairs * 2 <= dim, NVFP4_ERR_ARG, "nvfp4_comfy_rope: bad sizes");
    NVFP4_REQUIRE(aligned(rotation, 8), NVFP4_ERR_ALIGN, "nvfp4_comfy_rope: rotation table needs 8-byte alignment");
    comfy_rope_kernel<<<grid_for(rows * heads * dim, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(rotation), static_cast<uint16_t*>(out), rows, heads, dim,
        pairs, backward);
    return launch_status("nvfp4_comfy_rope");
}
