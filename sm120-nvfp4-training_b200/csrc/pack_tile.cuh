// Both NVFP4 orientations of one 128 x 128 tile of a contiguous weight matrix, as a device function: the second phase of
// the optimizer kernel that emits the next forward's weight packings (round to nearest, no Hadamard transform, one
// tensor scale for both orientations; the same bytes as nvfp4_quantize with pair = 1 on the updated weight).
//
// The source was written earlier in the same launch by other CTAs, so it is read with ld.global.cg (L2), never through
// the non-coherent path.
#pragma once
#include "quant_core.cuh"

namespace nvfp4 {

constexpr int PT_TILE = 128;
constexpr int PT_PITCH = PT_TILE + 8;     // bf16 elements per shared row (272 B keeps 16-byte alignment)
constexpr int PT_OUT_PITCH = 72;          // bytes per transposed payload row in shared memory

struct PackSmem {
    __align__(16) uint16_t tile[PT_TILE * PT_PITCH];
    __align__(16) uint8_t col_out[PT_TILE * PT_OUT_PITCH];
    __align__(16) uint8_t row_sc[1024];
    __align__(16) uint8_t col_sc[1024];
};

struct PackArgs {
    uint8_t* d; uint8_t* s; uint8_t* dt; uint8_t* st;   // row packing / scales, transposed packing / scales
    int64_t rows, cols;                                 // the weight is [rows][cols], contiguous
    unsigned int* barrier;                              // grid barrier word (zero between launches)
    int* status;                                        // nullable: raised when the barrier wait gave up
};

// 16 consecutive source elements of row r from column c0 as BF16 bit patterns (zero outside the matrix).
// MASTER: 32 FP32, 17 FP16, 16 / 24 BF16 (the BF16 head of a split master is the value the forward quantises).
template <int MASTER>
__device__ __forceinline__ void pack_load16(const void* w, int64_t r, int64_t c0, int64_t rows, int64_t cols, bool vec_ok, uint16_t (&h)[16]) {
    if (r >= rows || c0 >= cols) {
#pragma unroll
        for (int l = 0; l < 16; ++l) h[l] = 0;
        return;
    }
    const int64_t at = r * cols + c0;
    if (vec_ok && c0 + 16 <= cols) {
        if constexpr (MASTER == 32) {
            const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(w) + at);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 f = __ldcg(p + j);
                h[4 * j] = bf16_bits(f.x); h[4 * j + 1] = bf16_bits(f.y); h[4 * j + 2] = bf16_bits(f.z); h[4 * j + 3] = bf16_bits(f.w);
            }
        } else {
            const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(w) + at);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint4 u = __ldcg(p + j);
                const uint32_t word[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    uint16_t lo = static_cast<uint16_t>(word[t] & 0xffffu), hi = static_cast<uint16_t>(word[t] >> 16);
                    if constexpr (MASTER == 17) {
                        lo = bf16_bits(__half2float(__ushort_as_half(lo)));
                        hi = bf16_bits(__half2float(__ushort_as_half(hi)));
                    }
                    h[8 * j + 2 * t] = lo; h[8 * j + 2 * t + 1] = hi;
                }
            }
        }
        return;
    }
#pragma unroll
    for (int l = 0; l < 16; ++l) {
        uint16_t v = 0;
        if (c0 + l < cols) {
            if constexpr (MASTER == 32) v = bf16_bits(__ldcg(static_cast<const float*>(w) + at + l));
            else {
                v = __ldcg(static_cast<const uint16_t*>(w) + at + l);
                if constexpr (MASTER == 17) v = bf16_bits(__half2float(__ushort_as_half(v)));
            }
        }
        h[l] = v;
    }
}

// One tile (rt, ct) by a CTA of 256 threads.  inv = 1 / tensor scale.
template <int MASTER>
__device__ __forceinline__ void pack_tile(const void* w, const PackArgs& k, int64_t rt, int64_t ct, float inv, PackSmem& S) {
    const int tid = threadIdx.x;
    const int64_t r0 = rt * PT_TILE, c0 = ct * PT_TILE;
    const int64_t kp_r = round128(k.cols), kp_c = round128(k.rows);
    const bool vec_ok = (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (k.cols * (MASTER == 32 ? 4 : 2)) % 16 == 0;
    // phase A: a thread owns 4 row groups (16 consecutive columns of one row)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gi = tid + 256 * i;
        const int lr = gi >> 3, gc = gi & 7;
        const int64_t r = r0 + lr, c = c0 + gc * 16;
        uint16_t h[16];
        pack_load16<MASTER>(w, r, c, k.rows, k.cols, vec_ok, h);
        uint4 a, b;
        a.x = h[0] | (uint32_t(h[1]) << 16); a.y = h[2] | (uint32_t(h[3]) << 16);
        a.z = h[4] | (uint32_t(h[5]) << 16); a.w = h[6] | (uint32_t(h[7]) << 16);
        b.x = h[8] | (uint32_t(h[9]) << 16); b.y = h[10] | (uint32_t(h[11]) << 16);
        b.z = h[12] | (uint32_t(h[13]) << 16); b.w = h[14] | (uint32_t(h[15]) << 16);
        uint4* dst = reinterpret_cast<uint4*>(&S.tile[lr * PT_PITCH + gc * 16]);
        dst[0] = a; dst[1] = b;
        float v[16];
#pragma unroll
        for (int l = 0; l < 16; ++l) v[l] = bf16_value(h[l]);
        uint32_t sb;
        const uint2 p = encode16<SR_NONE, false>(v, false, inv, 0u, 0u, 0ull, sb);
        *reinterpret_cast<uint2*>(k.d + r * (kp_r >> 1) + (c >> 1)) = p;
        S.row_sc[(gc >> 2) * 512 + (lr & 31) * 16 + (lr >> 5) * 4 + (gc & 3)] = static_cast<uint8_t>(sb);
    }
    __syncthreads();
    if (tid < 64) {
        uint8_t* dst = k.s + (rt * (kp_r >> 6) + ct * 2) * 512;
        reinterpret_cast<uint4*>(dst)[tid] = reinterpret_cast<const uint4*>(S.row_sc)[tid];
    }
    // phase B: a thread takes two adjacent source columns and encodes source rows g*16 .. g*16+15 of each
    const int cp = tid & 63;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int g = (tid >> 6) + 4 * i;
        uint32_t wv[16];
#pragma unroll
        for (int l = 0; l < 16; ++l) wv[l] = *reinterpret_cast<const uint32_t*>(&S.tile[(g * 16 + l) * PT_PITCH + 2 * cp]);
#pragma unroll
        for (int side = 0; side < 2; ++side) {
            const int n = 2 * cp + side;
            float v[16];
#pragma unroll
            for (int l = 0; l < 16; ++l) v[l] = __uint_as_float(side ? (wv[l] & 0xffff0000u) : (wv[l] << 16));
            uint32_t sb;
            const uint2 p = encode16<SR_NONE, false>(v, false, inv, 0u, 0u, 0ull, sb);
            *reinterpret_cast<uint2*>(S.col_out + n * PT_OUT_PITCH + g * 8) = p;
            S.col_sc[(g >> 2) * 512 + (n & 31) * 16 + (n >> 5) * 4 + (g & 3)] = static_cast<uint8_t>(sb);
        }
    }
    __syncthreads();
    if (tid < 64) {
        uint8_t* dst = k.st + (ct * (kp_c >> 6) + rt * 2) * 512;
        reinterpret_cast<uint4*>(dst)[tid] = reinterpret_cast<const uint4*>(S.col_sc)[tid];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int ci = tid + 256 * i;
        const int nn = ci >> 3, ch = ci & 7;
        const uint2 p = *reinterpret_cast<const uint2*>(S.col_out + nn * PT_OUT_PITCH + ch * 8);
        *reinterpret_cast<uint2*>(k.dt + (c0 + nn) * (kp_c >> 1) + (r0 >> 1) + ch * 8) = p;
    }
    __syncthreads();   // the shared tile is free for the next one
}

}  // namespace nvfp4
