// Fused BF16 element-wise kernels of the decoder workload that sit between the NVFP4 layers: rotary position embedding
// and SwiGLU gating, forward and backward.  Pure HBM-bound streaming kernels: 16-byte vector loads and stores, FP32
// math, one rounding to BF16 at the end.  They replace chains of 4-6 generic tensor-iterator kernels per use.
#include "common.cuh"

#include <algorithm>

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

// x, out: [tokens = B*S][H][D] BF16 (row pitch `pitch` elements, heads contiguous); cos, sin: [S][D/2] BF16.
// out[.., j] = a cos - b sin, out[.., j + D/2] = b cos + a sin with (a, b) = (x[.., j], x[.., j + D/2]); sign = -1 inverts.
__global__ void __launch_bounds__(256) rope_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ out,
                                                   const uint16_t* __restrict__ cos_t, const uint16_t* __restrict__ sin_t,
                                                   int64_t tokens, int seq, int heads, int dim, int64_t pitch, float sign) {
    const int half = dim >> 1, chunks = half >> 3;   // 8 elements per thread from each half
    const int64_t total = tokens * heads * chunks;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % chunks);
        const int64_t th = i / chunks;
        const int h = static_cast<int>(th % heads);
        const int64_t t = th / heads;
        const int s = static_cast<int>(t % seq);
        const int64_t base = t * pitch + static_cast<int64_t>(h) * dim + c * 8;
        float a[8], b[8], cs[8], sn[8], ra[8], rb[8];
        unpack8(*reinterpret_cast<const uint4*>(x + base), a);
        unpack8(*reinterpret_cast<const uint4*>(x + base + half), b);
        unpack8(__ldg(reinterpret_cast<const uint4*>(cos_t + static_cast<int64_t>(s) * half + c * 8)), cs);
        unpack8(__ldg(reinterpret_cast<const uint4*>(sin_t + static_cast<int64_t>(s) * half + c * 8)), sn);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float sj = sn[j] * sign;
            ra[j] = a[j] * cs[j] - b[j] * sj;
            rb[j] = b[j] * cs[j] + a[j] * sj;
        }
        *reinterpret_cast<uint4*>(out + base) = pack8(ra);
        *reinterpret_cast<uint4*>(out + base + half) = pack8(rb);
    }
}

__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                                         uint4* __restrict__ out, int64_t chunks) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < chunks; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        float g[8], u[8], o[8];
        unpack8(gate[i], g); unpack8(up[i], u);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
        out[i] = pack8(o);
    }
}
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                                         const uint4* __restrict__ dout, uint4* __restrict__ dgate,
                                                         uint4* __restrict__ dup, int64_t chunks) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < chunks; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        float g[8], u[8], d[8], dg[8], du[8];
        unpack8(gate[i], g); unpack8(up[i], u); unpack8(dout[i], d);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float sg = 1.f / (1.f + __expf(-g[j]));
            const float silu = g[j] * sg;
            du[j] = d[j] * silu;
            dg[j] = d[j] * u[j] * (sg + silu * (1.f - sg));
        }
        dgate[i] = pack8(dg); dup[i] = pack8(du);
    }
}

static unsigned stream_grid(int64_t work_items) {
    return static_cast<unsigned>(std::min<int64_t>((work_items + 255) / 256, 148 * 16));
}

}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_rope(const void* x, void* out, const void* cos_t, const void* sin_t, int64_t tokens, int seq, int heads,
                          int dim, int64_t pitch, int inverse, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(x && out && cos_t && sin_t, NVFP4_ERR_ARG, "nvfp4_rope: null pointer");
    NVFP4_REQUIRE(tokens > 0 && seq > 0 && heads > 0 && dim > 0 && dim % 16 == 0 && pitch >= static_cast<int64_t>(heads) * dim && pitch % 8 == 0,
                  NVFP4_ERR_ARG, "nvfp4_rope: head dimension must be a multiple of 16 and the row pitch a multiple of 8");
    for (const void* p : {x, static_cast<const void*>(out), cos_t, sin_t})
        NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_rope: pointers must be 16-byte aligned");
    const int64_t items = tokens * heads * (dim / 16);
    rope_kernel<<<stream_grid(items), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), static_cast<const uint16_t*>(cos_t),
        static_cast<const uint16_t*>(sin_t), tokens, seq, heads, dim, pitch, inverse ? -1.f : 1.f);
    return launch_status("nvfp4_rope");
}

extern "C" int nvfp4_swiglu(const void* gate, const void* up, const void* dout, void* out_or_dgate, void* dup, int64_t n,
                            nvfp4_stream_t stream) {
    NVFP4_REQUIRE(gate && up && out_or_dgate && n > 0 && n % 8 == 0, NVFP4_ERR_ARG, "nvfp4_swiglu: null pointer or size not a multiple of 8");
    NVFP4_REQUIRE((dout == nullptr) == (dup == nullptr), NVFP4_ERR_ARG, "nvfp4_swiglu: backward needs both dout and dup");
    for (const void* p : {gate, up, dout, static_cast<const void*>(out_or_dgate), static_cast<const void*>(dup)})
        NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_swiglu: pointers must be 16-byte aligned");
    const int64_t chunks = n / 8;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dout) swiglu_bwd_kernel<<<stream_grid(chunks), 256, 0, st>>>(static_cast<const uint4*>(gate), static_cast<const uint4*>(up),
                                                                    static_cast<const uint4*>(dout), static_cast<uint4*>(out_or_dgate),
                                                                    static_cast<uint4*>(dup), chunks);
    else swiglu_fwd_kernel<<<stream_grid(chunks), 256, 0, st>>>(static_cast<const uint4*>(gate), static_cast<const uint4*>(up),
                                                               static_cast<uint4*>(out_or_dgate), chunks);
    return launch_status("nvfp4_swiglu");
}
