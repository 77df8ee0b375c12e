// Eight BF16 values in one 16-byte vector: unpack to FP32, pack with one rounding, magnitude maximum; warp reductions
// and the atomic maximum that leaves a tensor's amax on the device.  Shared by the element-wise and the loss kernels.
#pragma once
#include "common.cuh"

namespace nvfp4 {

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// max |v| of non-negative floats through their bit patterns (order-free, hence bit-identical to a separate amax pass)
__device__ __forceinline__ void atomic_amax(float* dst, float a) {
    if (dst && a > 0.f) atomicMax(reinterpret_cast<unsigned int*>(dst), __float_as_uint(a));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}
// One atomic per warp: for kernels whose few, long-running CTAs would otherwise wait for their slowest warp at the end.
__device__ __forceinline__ void warp_atomic_amax(float* dst, float best) {
    best = warp_max(best);
    if ((threadIdx.x & 31) == 0) atomic_amax(dst, best);
}
// One atomic per CTA: tens of thousands of same-address atomics (one per warp) serialise in the L2 and were measured to
// cost more than the kernel's data movement.  Every thread of the CTA must call it.
__device__ __forceinline__ void block_atomic_amax(float* dst, float best) {
    __shared__ float warp_best[32];
    best = warp_max(best);
    if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        float b = threadIdx.x < ((blockDim.x + 31) >> 5) ? warp_best[threadIdx.x] : 0.f;
        b = warp_max(b);
        if (threadIdx.x == 0) atomic_amax(dst, b);
    }
}
__device__ __forceinline__ float abs_max8(const uint4& packed) {   // max |bf16| of eight packed values
    const uint32_t w[4] = {packed.x, packed.y, packed.z, packed.w};
    uint32_t best = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) { best = max(best, w[i] & 0x7fffu); best = max(best, (w[i] >> 16) & 0x7fffu); }
    return __uint_as_float(best << 16);
}

}  // namespace nvfp4
