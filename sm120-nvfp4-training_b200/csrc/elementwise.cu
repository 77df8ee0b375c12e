// Fused BF16 element-wise kernels of the decoder workload that sit between the NVFP4 layers: rotary position embedding
// and SwiGLU gating, forward and backward.  Pure HBM-bound streaming kernels: 16-byte vector loads and stores, FP32
// math, one rounding to BF16 at the end.  They replace chains of 4-6 generic tensor-iterator kernels per use.
#include "common.cuh"
#include "bf16x8.cuh"

#include <algorithm>

namespace nvfp4 {

// x, out: [tokens = B*S][H][D] BF16 (row pitch `pitch` elements, heads contiguous); cos, sin: [S][D/2] BF16.
// out[.., j] = a cos - b sin, out[.., j + D/2] = b cos + a sin with (a, b) = (x[.., j], x[.., j + D/2]); sign = -1 inverts.
// sign = 0 copies (the third projection of a fused q / k / v gradient, which is not rotated).  amax (nullable) receives
// max |out|.
// Up to three tensors per launch (blockIdx.y picks one): the gradients of q, k and v go into one fused tensor this way.
struct RopeJobs {
    const uint16_t* x[3];
    uint16_t* out[3];
    int64_t pitch[3];
    float sign[3];
};
__global__ void __launch_bounds__(256) rope_kernel(const RopeJobs jobs, const uint16_t* __restrict__ cos_t,
                                                   const uint16_t* __restrict__ sin_t, int64_t tokens, int seq, int heads, int dim,
                                                   int64_t out_pitch, float* __restrict__ amax) {
    const int job = blockIdx.y;        // selected with conditionals: indexing a by-value struct would copy it to local memory
    const uint16_t* __restrict__ x = job == 0 ? jobs.x[0] : job == 1 ? jobs.x[1] : jobs.x[2];
    uint16_t* __restrict__ out = job == 0 ? jobs.out[0] : job == 1 ? jobs.out[1] : jobs.out[2];
    const int64_t pitch = job == 0 ? jobs.pitch[0] : job == 1 ? jobs.pitch[1] : jobs.pitch[2];
    const float sign = job == 0 ? jobs.sign[0] : job == 1 ? jobs.sign[1] : jobs.sign[2];
    float best = 0.f;
    const int half = dim >> 1, chunks = half >> 3;   // 8 elements per thread from each half
    const int64_t total = tokens * heads * chunks;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int c = static_cast<int>(i % chunks);
        const int64_t th = i / chunks;
        const int h = static_cast<int>(th % heads);
        const int64_t t = th / heads;
        const int s = static_cast<int>(t % seq);
        const int64_t base = t * pitch + static_cast<int64_t>(h) * dim + c * 8;
        const int64_t obase = t * out_pitch + static_cast<int64_t>(h) * dim + c * 8;
        uint4 pa = *reinterpret_cast<const uint4*>(x + base), pb = *reinterpret_cast<const uint4*>(x + base + half);
        if (sign != 0.f) {
            float a[8], b[8], cs[8], sn[8], ra[8], rb[8];
            unpack8(pa, a);
            unpack8(pb, b);
            unpack8(__ldg(reinterpret_cast<const uint4*>(cos_t + static_cast<int64_t>(s) * half + c * 8)), cs);
            unpack8(__ldg(reinterpret_cast<const uint4*>(sin_t + static_cast<int64_t>(s) * half + c * 8)), sn);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float sj = sn[j] * sign;
                ra[j] = a[j] * cs[j] - b[j] * sj;
                rb[j] = b[j] * cs[j] + a[j] * sj;
            }
            pa = pack8(ra); pb = pack8(rb);
        }
        *reinterpret_cast<uint4*>(out + obase) = pa;
        *reinterpret_cast<uint4*>(out + obase + half) = pb;
        if (amax) best = fmaxf(best, fmaxf(abs_max8(pa), abs_max8(pb)));
    }
    if (amax) block_atomic_amax(amax, best);
}

// gate, up, out (and dout, dgate, dup): [rows][cols] BF16 with their own row pitches (elements, multiples of 8), so that
// the two halves of a fused gate / up projection and of its gradient are addressed in place.  amax (nullable) receives
// max |out| (forward) or max over both gradients (backward).
struct Rows { const uint16_t* p; int64_t pitch; };
struct RowsOut { uint16_t* p; int64_t pitch; };
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(Rows gate, Rows up, RowsOut out, int64_t rows, int chunks, float* __restrict__ amax) {
    float best = 0.f;
    const int64_t total = rows * chunks;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / chunks;
        const int c = static_cast<int>(i - r * chunks) * 8;
        float g[8], u[8], o[8];
        unpack8(*reinterpret_cast<const uint4*>(gate.p + r * gate.pitch + c), g);
        unpack8(*reinterpret_cast<const uint4*>(up.p + r * up.pitch + c), u);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __fdividef(g[j], 1.f + __expf(-g[j])) * u[j];   // result is rounded to BF16: the fast quotient's 2 ulp do not show
        const uint4 packed = pack8(o);
        *reinterpret_cast<uint4*>(out.p + r * out.pitch + c) = packed;
        best = fmaxf(best, abs_max8(packed));
    }
    if (amax) block_atomic_amax(amax, best);
}
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(Rows gate, Rows up, Rows dout, RowsOut dgate, RowsOut dup, int64_t rows, int chunks,
                                                         float* __restrict__ amax) {
    float best = 0.f;
    const int64_t total = rows * chunks;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / chunks;
        const int c = static_cast<int>(i - r * chunks) * 8;
        float g[8], u[8], d[8], dg[8], du[8];
        unpack8(*reinterpret_cast<const uint4*>(gate.p + r * gate.pitch + c), g);
        unpack8(*reinterpret_cast<const uint4*>(up.p + r * up.pitch + c), u);
        unpack8(*reinterpret_cast<const uint4*>(dout.p + r * dout.pitch + c), d);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float sg = __fdividef(1.f, 1.f + __expf(-g[j]));
            const float silu = g[j] * sg;
            du[j] = d[j] * silu;
            dg[j] = d[j] * u[j] * (sg + silu * (1.f - sg));
        }
        const uint4 pg = pack8(dg), pu = pack8(du);
        *reinterpret_cast<uint4*>(dgate.p + r * dgate.pitch + c) = pg;
        *reinterpret_cast<uint4*>(dup.p + r * dup.pitch + c) = pu;
        best = fmaxf(best, fmaxf(abs_max8(pg), abs_max8(pu)));
    }
    if (amax) warp_atomic_amax(amax, best);   // measured: 118.6 us against 125.2 us with the CTA-level form, which helps the other kernels
}

static unsigned stream_grid(int64_t work_items) {
    return static_cast<unsigned>(std::min<int64_t>((work_items + 255) / 256, 148 * 16));
}

}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_rope(const void* x, void* out, const void* cos_t, const void* sin_t, int64_t tokens, int seq, int heads,
                          int dim, int64_t pitch, int64_t out_pitch, int mode, float* amax, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(x && out && (mode == 2 || (cos_t && sin_t)), NVFP4_ERR_ARG, "nvfp4_rope: null pointer");
    NVFP4_REQUIRE(mode >= 0 && mode <= 2, NVFP4_ERR_ARG, "nvfp4_rope: mode is 0 (rotate), 1 (inverse rotation) or 2 (copy)");
    const int64_t width = static_cast<int64_t>(heads) * dim;
    NVFP4_REQUIRE(tokens > 0 && seq > 0 && heads > 0 && dim > 0 && dim % 16 == 0 && pitch >= width && pitch % 8 == 0 &&
                  out_pitch >= width && out_pitch % 8 == 0, NVFP4_ERR_ARG,
                  "nvfp4_rope: head dimension must be a multiple of 16 and the row pitches multiples of 8");
    for (const void* p : {x, static_cast<const void*>(out), cos_t, sin_t})
        NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_rope: pointers must be 16-byte aligned");
    const int64_t items = tokens * heads * (dim / 16);
    RopeJobs jobs{};
    jobs.x[0] = static_cast<const uint16_t*>(x); jobs.out[0] = static_cast<uint16_t*>(out); jobs.pitch[0] = pitch;
    jobs.sign[0] = mode == 0 ? 1.f : mode == 1 ? -1.f : 0.f;
    rope_kernel<<<stream_grid(items), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        jobs, static_cast<const uint16_t*>(cos_t), static_cast<const uint16_t*>(sin_t), tokens, seq, heads, dim, out_pitch, amax);
    return launch_status("nvfp4_rope");
}

extern "C" int nvfp4_rope_qkv_bwd(const void* dq, int64_t dq_pitch, const void* dk, int64_t dk_pitch, const void* dv, int64_t dv_pitch,
                                  void* dqkv, const void* cos_t, const void* sin_t, int64_t tokens, int seq, int heads, int dim,
                                  float* amax, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(dq && dk && dv && dqkv && cos_t && sin_t, NVFP4_ERR_ARG, "nvfp4_rope_qkv_bwd: null pointer");
    const int64_t width = static_cast<int64_t>(heads) * dim;
    NVFP4_REQUIRE(tokens > 0 && seq > 0 && heads > 0 && dim > 0 && dim % 16 == 0, NVFP4_ERR_ARG,
                  "nvfp4_rope_qkv_bwd: head dimension must be a multiple of 16");
    for (int64_t pitch : {dq_pitch, dk_pitch, dv_pitch})
        NVFP4_REQUIRE(pitch >= width && pitch % 8 == 0, NVFP4_ERR_ARG, "nvfp4_rope_qkv_bwd: row pitches must be multiples of 8, at least heads * dim");
    for (const void* p : {dq, dk, dv, static_cast<const void*>(dqkv), cos_t, sin_t})
        NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_rope_qkv_bwd: pointers must be 16-byte aligned");
    RopeJobs jobs{};
    const void* src[3] = {dq, dk, dv};
    const int64_t pitches[3] = {dq_pitch, dk_pitch, dv_pitch};
    for (int i = 0; i < 3; ++i) {
        jobs.x[i] = static_cast<const uint16_t*>(src[i]);
        jobs.out[i] = static_cast<uint16_t*>(dqkv) + width * i;
        jobs.pitch[i] = pitches[i];
        jobs.sign[i] = i < 2 ? -1.f : 0.f;          // inverse rotation of dq and dk, copy of dv
    }
    const int64_t items = tokens * heads * (dim / 16);
    dim3 grid(stream_grid(items), 3);
    rope_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        jobs, static_cast<const uint16_t*>(cos_t), static_cast<const uint16_t*>(sin_t), tokens, seq, heads, dim, 3 * width, amax);
    return launch_status("nvfp4_rope_qkv_bwd");
}

extern "C" int nvfp4_swiglu(const void* gate, int64_t gate_pitch, const void* up, int64_t up_pitch, const void* dout, int64_t dout_pitch,
                            void* out_or_dgate, int64_t out_pitch, void* dup, int64_t dup_pitch, int64_t rows, int64_t cols,
                            float* amax, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(gate && up && out_or_dgate && rows > 0 && cols > 0 && cols % 8 == 0, NVFP4_ERR_ARG,
                  "nvfp4_swiglu: null pointer or column count not a multiple of 8");
    NVFP4_REQUIRE((dout == nullptr) == (dup == nullptr), NVFP4_ERR_ARG, "nvfp4_swiglu: backward needs both dout and dup");
    for (int64_t pitch : {gate_pitch, up_pitch, out_pitch, dout ? dout_pitch : cols, dup ? dup_pitch : cols})
        NVFP4_REQUIRE(pitch >= cols && pitch % 8 == 0, NVFP4_ERR_ARG, "nvfp4_swiglu: row pitches must be multiples of 8, at least the column count");
    for (const void* p : {gate, up, dout, static_cast<const void*>(out_or_dgate), static_cast<const void*>(dup)})
        NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_swiglu: pointers must be 16-byte aligned");
    const int chunks = static_cast<int>(cols / 8);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const Rows g{static_cast<const uint16_t*>(gate), gate_pitch}, u{static_cast<const uint16_t*>(up), up_pitch};
    if (dout) swiglu_bwd_kernel<<<stream_grid(rows * chunks), 256, 0, st>>>(g, u, Rows{static_cast<const uint16_t*>(dout), dout_pitch},
                                                                           RowsOut{static_cast<uint16_t*>(out_or_dgate), out_pitch},
                                                                           RowsOut{static_cast<uint16_t*>(dup), dup_pitch}, rows, chunks, amax);
    else swiglu_fwd_kernel<<<stream_grid(rows * chunks), 256, 0, st>>>(g, u, RowsOut{static_cast<uint16_t*>(out_or_dgate), out_pitch}, rows, chunks, amax);
    return launch_status("nvfp4_swiglu");
}

// ====================================================================================================================
// Residual add + RMSNorm, forward and backward, with the tensor amax of what the next NVFP4 layer will quantise
// ====================================================================================================================
namespace nvfp4 {

// One warp per token row.  sum = bf16(x + delta) (written when delta is given), h = bf16(sum * rstd * bf16(gamma)),
// rstd = rsqrt(mean(sum^2) + eps) kept in FP32 for the backward pass.  The row stays in shared memory between the two
// sweeps, so x and delta are read once.
__global__ void __launch_bounds__(256) add_rmsnorm_fwd_kernel(const uint4* __restrict__ x, const uint4* __restrict__ delta,
                                                              const float* __restrict__ gamma, float eps, int64_t rows, int chunks,
                                                              uint4* __restrict__ sum_out, uint4* __restrict__ h_out,
                                                              float* __restrict__ rstd_out, float* __restrict__ amax_out) {
    extern __shared__ uint4 row_cache[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    uint4* mine = row_cache + static_cast<size_t>(warp) * chunks;
    float best = 0.f;
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * warps + warp; r < rows; r += static_cast<int64_t>(gridDim.x) * warps) {
        const uint4* xr = x + r * chunks;
        float sq = 0.f;
#pragma unroll 4
        for (int c = lane; c < chunks; c += 32) {
            uint4 v = xr[c];
            if (delta) {
                float a[8], b[8];
                unpack8(v, a); unpack8(delta[r * chunks + c], b);
#pragma unroll
                for (int j = 0; j < 8; ++j) a[j] += b[j];
                v = pack8(a);
                sum_out[r * chunks + c] = v;
            }
            float f[8];
            unpack8(v, f);
#pragma unroll
            for (int j = 0; j < 8; ++j) sq = fmaf(f[j], f[j], sq);
            mine[c] = v;
        }
        sq = warp_sum(sq);
        const float rstd = rsqrtf(sq / static_cast<float>(chunks * 8) + eps);
        if (lane == 0) rstd_out[r] = rstd;
        __syncwarp();
        for (int c = lane; c < chunks; c += 32) {
            float f[8], g[8];
            unpack8(mine[c], f);
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c), g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c + 1);
            g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * bf16_value(bf16_bits(g[j]));
            const uint4 o = pack8(f);
            h_out[r * chunks + c] = o;
            best = fmaxf(best, abs_max8(o));
        }
        __syncwarp();
    }
    warp_atomic_amax(amax_out, best);
}

// Backward of h = sum * rstd * gamma for one warp per row, plus the gradient that arrives on the residual path:
//   u = dh * gamma, dx = rstd * u - sum * (rstd^3 / D) * <u, sum> + dres.
// dgamma needs a sum over all rows: every warp keeps its own FP32 column accumulators in shared memory, the CTA adds its
// warps in a fixed order and writes one partial row; colsum_finish_kernel adds the partial rows in a fixed order, so the
// result does not depend on scheduling.
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const uint4* __restrict__ dh, const uint4* __restrict__ sum,
                                                          const float* __restrict__ rstd, const float* __restrict__ gamma,
                                                          const uint4* __restrict__ dres, int64_t rows, int chunks,
                                                          uint4* __restrict__ dx, float* __restrict__ partial,
                                                          float* __restrict__ amax_out) {
    extern __shared__ uint4 row_cache[];
    float* acc = reinterpret_cast<float*>(row_cache);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int cols = chunks * 8;
    float* mine = acc + static_cast<size_t>(warp) * cols;
    for (int j = lane; j < cols; j += 32) mine[j] = 0.f;
    __syncwarp();
    const float inv_d = 1.f / static_cast<float>(cols);
    float best = 0.f;
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * warps + warp; r < rows; r += static_cast<int64_t>(gridDim.x) * warps) {
        const float rs = rstd[r];
        float dot = 0.f;
#pragma unroll 4
        for (int c = lane; c < chunks; c += 32) {
            float g[8], s[8], w[8];
            unpack8(dh[r * chunks + c], g); unpack8(sum[r * chunks + c], s);
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c), g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c + 1);
            w[0] = g0.x; w[1] = g0.y; w[2] = g0.z; w[3] = g0.w; w[4] = g1.x; w[5] = g1.y; w[6] = g1.z; w[7] = g1.w;
            float* a = mine + c * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                dot = fmaf(g[j] * bf16_value(bf16_bits(w[j])), s[j], dot);
                a[j] = fmaf(g[j] * s[j], rs, a[j]);
            }
        }
        dot = warp_sum(dot);
        const float k = rs * rs * rs * inv_d * dot;
#pragma unroll 4
        for (int c = lane; c < chunks; c += 32) {
            float g[8], s[8], w[8], o[8];
            unpack8(dh[r * chunks + c], g); unpack8(sum[r * chunks + c], s);
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c), g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c + 1);
            w[0] = g0.x; w[1] = g0.y; w[2] = g0.z; w[3] = g0.w; w[4] = g1.x; w[5] = g1.y; w[6] = g1.z; w[7] = g1.w;
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = rs * (g[j] * bf16_value(bf16_bits(w[j]))) - s[j] * k;
            if (dres) {
                float d[8];
                unpack8(dres[r * chunks + c], d);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] += d[j];
            }
            const uint4 packed = pack8(o);
            dx[r * chunks + c] = packed;
            best = fmaxf(best, abs_max8(packed));
        }
    }
    block_atomic_amax(amax_out, best);
    __syncthreads();
    for (int j = threadIdx.x; j < cols; j += blockDim.x) {
        float t = 0.f;
        for (int w = 0; w < warps; ++w) t += acc[static_cast<size_t>(w) * cols + j];
        partial[static_cast<size_t>(blockIdx.x) * cols + j] = t;
    }
}

// The same backward pass with every thread owning CPT fixed groups of eight columns: the dgamma sums stay in registers,
// RB_ROWS rows are in flight per thread (all of their loads are issued before the first is used; two CTAs per SM alternate between
// loading and computing) and each row is read once.
// The row-wise dot products are combined through shared memory in a fixed order.  Used when the column count divides
// evenly over the CTA; the warp-per-row kernel above serves the other shapes.
constexpr int RB_ROWS = 2;   // rows in flight per thread of the column-owner kernel

template <int CPT>
__global__ void __launch_bounds__(384, CPT == 1 ? 2 : 1) rmsnorm_bwd_cols_kernel(const uint4* __restrict__ dh, const uint4* __restrict__ sum,
                                                               const float* __restrict__ rstd, const float* __restrict__ gamma,
                                                               const uint4* __restrict__ dres, int64_t rows, int chunks,
                                                               uint4* __restrict__ dx, float* __restrict__ partial,
                                                               float* __restrict__ amax_out) {
    constexpr int R = RB_ROWS;
    __shared__ float dots[2][R][12];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
    float w[CPT][8], acc[CPT][8];
#pragma unroll
    for (int k = 0; k < CPT; ++k) {
        const int c = tid + k * blockDim.x;
        const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c), g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c + 1);
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) { w[k][j] = bf16_value(bf16_bits(g[j])); acc[k][j] = 0.f; }
    }
    const float inv_d = 1.f / static_cast<float>(chunks * 8);
    float best = 0.f;
    int phase = 0;
    for (int64_t r0 = static_cast<int64_t>(blockIdx.x) * R; r0 < rows; r0 += static_cast<int64_t>(gridDim.x) * R, phase ^= 1) {
        uint4 pg[R][CPT], ps[R][CPT], pd[R][CPT];   // the residual-path gradient is fetched with the other two operands
#pragma unroll
        for (int i = 0; i < R; ++i)
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const int64_t at = (r0 + i) * chunks + tid + k * blockDim.x;
                const bool live = r0 + i < rows;
                pg[i][k] = live ? dh[at] : make_uint4(0, 0, 0, 0);
                ps[i][k] = live ? sum[at] : make_uint4(0, 0, 0, 0);
                pd[i][k] = (live && dres) ? dres[at] : make_uint4(0, 0, 0, 0);
            }
        float rs[R], dot[R];
#pragma unroll
        for (int i = 0; i < R; ++i) {
            rs[i] = r0 + i < rows ? rstd[r0 + i] : 0.f;
            dot[i] = 0.f;
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                float g[8], sv[8];
                unpack8(pg[i][k], g); unpack8(ps[i][k], sv);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    dot[i] = fmaf(g[j] * w[k][j], sv[j], dot[i]);
                    acc[k][j] = fmaf(g[j] * sv[j], rs[i], acc[k][j]);
                }
            }
            dot[i] = warp_sum(dot[i]);
            if (lane == 0) dots[phase][i][warp] = dot[i];
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < R; ++i) {
            if (r0 + i >= rows) break;
            float total = 0.f;
            for (int q = 0; q < warps; ++q) total += dots[phase][i][q];
            const float kf = rs[i] * rs[i] * rs[i] * inv_d * total;
#pragma unroll
            for (int k = 0; k < CPT; ++k) {
                const int64_t at = (r0 + i) * chunks + tid + k * blockDim.x;
                float g[8], sv[8], o[8];
                unpack8(pg[i][k], g); unpack8(ps[i][k], sv);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = rs[i] * (g[j] * w[k][j]) - sv[j] * kf;
                if (dres) {
                    float d[8];
                    unpack8(pd[i][k], d);
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] += d[j];
                }
                const uint4 packed = pack8(o);
                dx[at] = packed;
                best = fmaxf(best, abs_max8(packed));
            }
        }
    }
    block_atomic_amax(amax_out, best);
#pragma unroll
    for (int k = 0; k < CPT; ++k) {
        float* dst = partial + static_cast<size_t>(blockIdx.x) * chunks * 8 + static_cast<size_t>(tid + k * blockDim.x) * 8;
        reinterpret_cast<float4*>(dst)[0] = make_float4(acc[k][0], acc[k][1], acc[k][2], acc[k][3]);
        reinterpret_cast<float4*>(dst)[1] = make_float4(acc[k][4], acc[k][5], acc[k][6], acc[k][7]);
    }
}

// Column sums of the per-CTA partial rows, in a fixed order: a CTA takes 32 columns, its eight warps take every eighth
// partial row each, and the eight subtotals are added in warp order.
__global__ void __launch_bounds__(256) colsum_finish_kernel(const float* __restrict__ partial, int parts, int cols, float* __restrict__ out) {
    __shared__ float subtotal[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = blockIdx.x * 32 + lane;
    float t = 0.f;
    if (j < cols) {
#pragma unroll 8
        for (int p = warp; p < parts; p += 8) t += partial[static_cast<size_t>(p) * cols + j];
    }
    subtotal[warp][lane] = t;
    __syncthreads();
    if (warp == 0 && j < cols) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) total += subtotal[w][lane];
        out[j] = total;
    }
}

}  // namespace nvfp4

static int norm_warps(int cols, int bytes_per_col) {   // warps per CTA whose row buffers fit 96 KB of shared memory
    int w = 8;
    while (w > 1 && static_cast<int64_t>(w) * cols * bytes_per_col > 96 * 1024) w >>= 1;
    return w;
}

extern "C" int nvfp4_add_rmsnorm(const void* x, const void* delta, const float* gamma, float eps, int64_t rows, int64_t cols,
                                 void* sum_out, void* h_out, float* rstd_out, float* amax_out, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(x && gamma && h_out && rstd_out, NVFP4_ERR_ARG, "nvfp4_add_rmsnorm: null pointer");
    NVFP4_REQUIRE(!delta || sum_out, NVFP4_ERR_ARG, "nvfp4_add_rmsnorm: the sum needs an output when a second operand is given");
    NVFP4_REQUIRE(rows > 0 && cols > 0 && cols % 8 == 0 && cols <= 49152, NVFP4_ERR_ARG, "nvfp4_add_rmsnorm: columns must be a multiple of 8, at most 49152");
    for (const void* p : {x, delta, static_cast<const void*>(gamma), static_cast<const void*>(sum_out), static_cast<const void*>(h_out)})
        NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_add_rmsnorm: pointers must be 16-byte aligned");
    const int warps = norm_warps(static_cast<int>(cols), 2);
    const size_t smem = static_cast<size_t>(warps) * cols * 2;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(add_rmsnorm_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        configured = true;
    }
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>((rows + warps - 1) / warps, 148 * 8));
    add_rmsnorm_fwd_kernel<<<grid, warps * 32, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(x), static_cast<const uint4*>(delta), gamma, eps, rows, static_cast<int>(cols / 8),
        static_cast<uint4*>(sum_out), static_cast<uint4*>(h_out), rstd_out, amax_out);
    return launch_status("nvfp4_add_rmsnorm");
}

// threads (a multiple of 32, at most 384) and column groups per thread (at most 2) of the column-owner kernel, or 0
static int cols_threads(int64_t cols, int* cpt) {
    const int64_t chunks = cols / 8;
    for (int k = 1; k <= 2; ++k)
        if (chunks % k == 0 && (chunks / k) % 32 == 0 && chunks / k <= 384) { *cpt = k; return static_cast<int>(chunks / k); }
    return 0;
}

extern "C" int64_t nvfp4_rmsnorm_bwd_partials(int64_t rows, int64_t cols) {
    int cpt = 0;
    if (cols_threads(cols, &cpt)) return std::min<int64_t>((rows + RB_ROWS - 1) / RB_ROWS, 148 * 2);
    const int warps = norm_warps(static_cast<int>(cols), 4);
    return std::min<int64_t>((rows + warps - 1) / warps, 148 * 2);
}

extern "C" int nvfp4_rmsnorm_bwd(const void* dh, const void* sum, const float* rstd, const float* gamma, const void* dres,
                                 int64_t rows, int64_t cols, void* dx, float* partial, float* dgamma, float* amax_out,
                                 nvfp4_stream_t stream) {
    NVFP4_REQUIRE(dh && sum && rstd && gamma && dx && partial && dgamma, NVFP4_ERR_ARG, "nvfp4_rmsnorm_bwd: null pointer");
    NVFP4_REQUIRE(rows > 0 && cols > 0 && cols % 8 == 0 && cols <= 24576, NVFP4_ERR_ARG, "nvfp4_rmsnorm_bwd: columns must be a multiple of 8, at most 24576");
    for (const void* p : {dh, sum, dres, static_cast<const void*>(gamma), static_cast<const void*>(dx)})
        NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_rmsnorm_bwd: pointers must be 16-byte aligned");
    const int warps = norm_warps(static_cast<int>(cols), 4);
    const size_t smem = static_cast<size_t>(warps) * cols * 4;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        configured = true;
    }
    const int parts = static_cast<int>(nvfp4_rmsnorm_bwd_partials(rows, cols));
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int cpt = 0;
    if (const int threads = cols_threads(cols, &cpt)) {
        auto launch = [&](auto kernel) {
            kernel<<<parts, threads, 0, st>>>(static_cast<const uint4*>(dh), static_cast<const uint4*>(sum), rstd, gamma,
                                             static_cast<const uint4*>(dres), rows, static_cast<int>(cols / 8), static_cast<uint4*>(dx),
                                             partial, amax_out);
        };
        if (cpt == 1) launch(rmsnorm_bwd_cols_kernel<1>);
        else launch(rmsnorm_bwd_cols_kernel<2>);
        colsum_finish_kernel<<<static_cast<unsigned>((cols + 31) / 32), 256, 0, st>>>(partial, parts, static_cast<int>(cols), dgamma);
        return launch_status("nvfp4_rmsnorm_bwd");
    }
    rmsnorm_bwd_kernel<<<parts, warps * 32, smem, st>>>(static_cast<const uint4*>(dh), static_cast<const uint4*>(sum), rstd, gamma,
                                                        static_cast<const uint4*>(dres), rows, static_cast<int>(cols / 8),
                                                        static_cast<uint4*>(dx), partial, amax_out);
    colsum_finish_kernel<<<static_cast<unsigned>((cols + 31) / 32), 256, 0, st>>>(partial, parts, static_cast<int>(cols), dgamma);
    return launch_status("nvfp4_rmsnorm_bwd");
}
