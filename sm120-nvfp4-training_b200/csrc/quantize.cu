// NVFP4 quantiser for sm_100a: tensor amax, tile quantiser (row packing and/or transposed packing
// from one read of the source), dequantiser.
//
// Numerical contract (bit exact against the CPU oracle): value = float(bf16_rne(x)); optional
// sign * H16 / 4 butterfly over the 16 contraction elements; block scale
// e4m3_rn(clamp((amax16 / 6) * (1 / pts), 2^-6, 448)); element q = clamp(v * ((1/pts) / scale), -6, 6)
// rounded to e2m1 by the hardware cvt.rn.satfinite or stochastically between adjacent levels.
// All float operations that take part in the contract are written with the _rn intrinsics so the
// compiler can never contract them into FMAs.
#include "common.cuh"

#include <cstdarg>
#include <cstring>
#include <cstddef>
#include <algorithm>

namespace nvfp4 {

static thread_local char g_error[512] = "";
void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}
int launch_status(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: CUDA launch failed: %s", what, cudaGetErrorString(e));
        return NVFP4_ERR_LAUNCH;
    }
    return NVFP4_OK;
}

// ================================================================================================
// amax
// ================================================================================================
constexpr int AMAX_MAX_BLOCKS = 1024;
constexpr int AMAX_THREADS = 256;
struct AmaxScratch {
    float partial[AMAX_MAX_BLOCKS];
    unsigned int ticket;  // starts at zero; the last block to arrive resets it
    unsigned int pad[3];
};

__device__ __forceinline__ float block_max_256(float a) {
    __shared__ float warp_max[8];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = a;
    __syncthreads();
    a = warp_max[threadIdx.x & 7];
#pragma unroll
    for (int d = 4; d > 0; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
    __syncthreads();
    return a;
}

template <int DT>
__device__ __forceinline__ float abs_max_of_chunk(uint4 q) {
    float a = 0.f;
    if constexpr (DT == NVFP4_F32) {
        a = fmaxf(fmaxf(fabsf(__uint_as_float(q.x)), fabsf(__uint_as_float(q.y))),
                  fmaxf(fabsf(__uint_as_float(q.z)), fabsf(__uint_as_float(q.w))));
    } else if constexpr (DT == NVFP4_BF16) {
        // |bf16| ordering equals the ordering of the 15 magnitude bits
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t best = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            best = max(best, w[i] & 0x7fffu);
            best = max(best, (w[i] >> 16) & 0x7fffu);
        }
        a = __uint_as_float(best << 16);
    } else {
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t best = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            best = max(best, w[i] & 0x7fffu);
            best = max(best, (w[i] >> 16) & 0x7fffu);
        }
        a = __half2float(__ushort_as_half(static_cast<unsigned short>(best)));
    }
    return a;
}

// Rounding to bf16 is monotonic, so max|bf16(x)| = bf16(max|x|): the reduction runs on raw magnitudes.
template <int DT>
__global__ void __launch_bounds__(AMAX_THREADS) amax_kernel(const void* __restrict__ x, int64_t rows, int64_t cols,
                                                           int64_t rs, int64_t cs, int dense_vec,
                                                           AmaxScratch* scratch, float* __restrict__ out4,
                                                           float* __restrict__ pts_dst, int which) {
    float a = 0.f;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
    if (dense_vec) {
        constexpr int PER = 16 / ElemSize<DT>::value;
        const int64_t n = rows * cols, nchunk = n / PER;
        const uint4* xv = static_cast<const uint4*>(x);
        for (int64_t i = tid; i < nchunk; i += nthreads) a = fmaxf(a, abs_max_of_chunk<DT>(__ldg(xv + i)));
        for (int64_t i = nchunk * PER + tid; i < n; i += nthreads) a = fmaxf(a, load_abs<DT>(x, i));
    } else {
        const int64_t n = rows * cols;
        for (int64_t i = tid; i < n; i += nthreads) {
            int64_t r = i / cols, c = i - r * cols;
            a = fmaxf(a, load_abs<DT>(x, r * rs + c * cs));
        }
    }
    a = block_max_256(a);
    __shared__ bool last;
    if (threadIdx.x == 0) {
        scratch->partial[blockIdx.x] = a;
        __threadfence();
        unsigned int t = atomicAdd(&scratch->ticket, 1u);
        last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    float b = 0.f;
    for (int i = threadIdx.x; i < static_cast<int>(gridDim.x); i += blockDim.x)
        b = fmaxf(b, *(volatile float*)&scratch->partial[i]);
    b = block_max_256(b);
    if (threadIdx.x == 0) {
        b = bf16_value(bf16_bits(b));
        const float c = 1.f / (6.f * 448.f);
        const float floor_a = fmaxf(b, 1.e-12f);
        out4[0] = b;
        out4[1] = __fmul_rn(__fmul_rn(1.f, floor_a), c);
        out4[2] = __fmul_rn(__fmul_rn(4.f, floor_a), c);
        out4[3] = __fdiv_rn(floor_a, 2688.f);
        if (pts_dst) *pts_dst = out4[which];
        scratch->ticket = 0u;
    }
}

// ================================================================================================
// group encoder
// ================================================================================================
// sign * H16 butterfly WITHOUT the final 1/4: that power-of-two factor is folded into the block
// amax and the element multiplier by the caller, which gives the same bits as scaling the 16 values
// first (a multiplication by 0.25 is exact).  The first stage absorbs the signs: a product with +-1
// is exact, so fma(b, s_b, a * s_a) rounds once, exactly like (a * s_a) + (b * s_b).
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

// Encodes 16 values (times `fold` = 0.25 when they come from hadamard16_unscaled, else 1).
// idx0 = flat index of element 0 in the packing's padded coordinates (a multiple of 16).
template <int SR>
__device__ __forceinline__ uint2 encode16(const float (&v)[16], bool fold, float inv_pts, bool hi_first, uint32_t seed,
                                          uint64_t idx0, uint32_t& scale_byte) {
    float a = 0.f;
#pragma unroll
    for (int l = 0; l < 16; ++l) a = fmaxf(a, fabsf(v[l]));
    if (fold) a = __fmul_rn(a, 0.25f);
    const float enc = fminf(fmaxf(__fmul_rn(__fdiv_rn(a, 6.f), inv_pts), 0.015625f), 448.f);
    const uint32_t e8 = __nv_cvt_float_to_fp8(enc, __NV_SATFINITE, __NV_E4M3);
    scale_byte = e8;
    float mul = __fdiv_rn(inv_pts, e4m3_normal_to_float(e8));
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
        // cvt.rn.satfinite clamps to +-6 by itself
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float q0 = q[2 * b], q1 = q[2 * b + 1], q2 = q[8 + 2 * b], q3 = q[8 + 2 * b + 1];
            const float2 p0 = hi_first ? make_float2(q1, q0) : make_float2(q0, q1);
            const float2 p1 = hi_first ? make_float2(q3, q2) : make_float2(q2, q3);
            lo |= static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(p0, __NV_E2M1, cudaRoundNearest)) << (8 * b);
            hi |= static_cast<uint32_t>(__nv_cvt_float2_to_fp4x2(p1, __NV_E2M1, cudaRoundNearest)) << (8 * b);
        }
        return make_uint2(lo, hi);
    } else {
        uint32_t codes[16];
        uint32_t rnd[8];
        if constexpr (SR == SR_PHILOX) {
            const uint64_t c0 = idx0 >> 3;  // one Philox block serves 8 consecutive elements (16 bits each)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint64_t ci = c0 + j;
                const uint4 r = philox4x32_10(make_uint4(static_cast<uint32_t>(ci), static_cast<uint32_t>(ci >> 32), 0u, 0u),
                                              seed, PHILOX_KEY1);
                rnd[4 * j] = r.x; rnd[4 * j + 1] = r.y; rnd[4 * j + 2] = r.z; rnd[4 * j + 3] = r.w;
            }
        }
        const uint32_t hbase = seed * 0x9e3779b9u + static_cast<uint32_t>(idx0) + 0x85ebca6bu;
#pragma unroll
        for (int l = 0; l < 16; ++l) {
            const float ql = q[l];
            // complement of the 24 random bits (the level choice adds it); Philox: 16-bit uniform on the 24-bit grid,
            // whose complement is (~r16 << 8) | 0xff
            uint32_t nh, bias = 0u;
            if constexpr (SR == SR_HASH) nh = shr_mul(~hash32_mixed(hbase + l), 1u << 24);
            else { nh = ((~rnd[l >> 1] >> ((l & 1) * 16)) & 0xffffu) << 8; bias = 0xffu; }
            codes[l] = sr_code_signed(ql, nh, bias);   // sign bit set iff q < 0 (so -0 encodes as +0)
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t e0 = codes[2 * b], o0 = codes[2 * b + 1], e1 = codes[8 + 2 * b], o1 = codes[8 + 2 * b + 1];
            lo |= (hi_first ? ((e0 << 4) | o0) : (e0 | (o0 << 4))) << (8 * b);
            hi |= (hi_first ? ((e1 << 4) | o1) : (e1 | (o1 << 4))) << (8 * b);
        }
        return make_uint2(lo, hi);
    }
}

// ================================================================================================
// tile quantiser: 128 x 128 source tile per CTA, 256 threads
// ================================================================================================
struct Orient {
    uint8_t* packed;
    uint8_t* scales;
    const float* pts;
    int64_t kp;  // padded contraction extent of this packing
    uint32_t seed;
    int flags;
};

constexpr int TILE = 128;
constexpr int TILE_PITCH = TILE + 8;  // bf16 elements per smem row (272 B keeps 16-byte alignment)
constexpr int COL_OUT_PITCH = 72;     // bytes per transposed payload row in smem (64 + 8: conflict-free 8-byte stores)

template <int DT>
__device__ __forceinline__ void load_group_bf16(const void* x, int64_t r, int64_t c0, int64_t rows, int64_t cols,
                                                int64_t rs, int64_t cs, bool vec_ok, uint16_t (&h)[16]) {
    if (r >= rows || c0 >= cols) {
#pragma unroll
        for (int l = 0; l < 16; ++l) h[l] = 0;
        return;
    }
    if (vec_ok && c0 + 16 <= cols) {
        if constexpr (DT == NVFP4_F32) {
            const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) + r * rs + c0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 f = __ldg(p + j);
                h[4 * j] = bf16_bits(f.x); h[4 * j + 1] = bf16_bits(f.y);
                h[4 * j + 2] = bf16_bits(f.z); h[4 * j + 3] = bf16_bits(f.w);
            }
        } else {
            const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + r * rs + c0);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint4 u = __ldg(p + j);
                uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    uint16_t lo = static_cast<uint16_t>(w[t] & 0xffffu), hi = static_cast<uint16_t>(w[t] >> 16);
                    if constexpr (DT == NVFP4_F16) {
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
    for (int l = 0; l < 16; ++l) h[l] = (c0 + l < cols) ? load_as_bf16<DT>(x, r * rs + (c0 + l) * cs) : uint16_t(0);
}

template <int DT, bool ROW, bool COL, int SR>
__global__ void __launch_bounds__(256, 4) quant_tile_kernel(const void* __restrict__ x, int64_t rows, int64_t cols,
                                                         int64_t rs, int64_t cs, int vec_ok,
                                                         const float* __restrict__ signs,
                                                         const int32_t* __restrict__ seed_base, Orient R, Orient C) {
    __shared__ __align__(16) uint16_t tile[COL ? TILE * TILE_PITCH : 8];
    __shared__ __align__(16) uint8_t row_sc[ROW ? 1024 : 16];
    __shared__ __align__(16) uint8_t col_sc[COL ? 1024 : 16];
    __shared__ __align__(16) uint8_t col_out[COL ? TILE * COL_OUT_PITCH : 16];

    const int tid = threadIdx.x;
    const int64_t rt = blockIdx.x, ct = blockIdx.y;
    const int64_t r0 = rt * TILE, c0 = ct * TILE;
    float sg[16];
#pragma unroll
    for (int l = 0; l < 16; ++l) sg[l] = __ldg(signs + l);
    const uint32_t base = seed_base ? static_cast<uint32_t>(__ldg(seed_base)) : 0u;

    float inv_r = 0.f;
    if constexpr (ROW) inv_r = __fdiv_rn(1.f, __ldg(R.pts));

    // ---- phase A: each thread owns 4 row groups (16 consecutive columns of one row) ----------------
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gi = tid + 256 * i;
        const int lr = gi >> 3, gc = gi & 7;
        const int64_t r = r0 + lr, c = c0 + gc * 16;
        uint16_t h[16];
        load_group_bf16<DT>(x, r, c, rows, cols, rs, cs, vec_ok != 0, h);
        if constexpr (COL) {
            uint4 a, b;
            a.x = h[0] | (uint32_t(h[1]) << 16); a.y = h[2] | (uint32_t(h[3]) << 16);
            a.z = h[4] | (uint32_t(h[5]) << 16); a.w = h[6] | (uint32_t(h[7]) << 16);
            b.x = h[8] | (uint32_t(h[9]) << 16); b.y = h[10] | (uint32_t(h[11]) << 16);
            b.z = h[12] | (uint32_t(h[13]) << 16); b.w = h[14] | (uint32_t(h[15]) << 16);
            uint4* dst = reinterpret_cast<uint4*>(&tile[lr * TILE_PITCH + gc * 16]);
            dst[0] = a; dst[1] = b;
        }
        if constexpr (ROW) {
            float v[16];
#pragma unroll
            for (int l = 0; l < 16; ++l) v[l] = bf16_value(h[l]);
            const bool rht = R.flags & NVFP4_Q_RHT;
            if (rht) hadamard16_unscaled(v, sg);
            uint32_t sb;
            uint2 p = encode16<SR>(v, rht, inv_r, R.flags & NVFP4_Q_HI_FIRST, R.seed + base,
                                   static_cast<uint64_t>(r) * R.kp + c, sb);
            *reinterpret_cast<uint2*>(R.packed + r * (R.kp >> 1) + (c >> 1)) = p;
            row_sc[(gc >> 2) * 512 + (lr & 31) * 16 + (lr >> 5) * 4 + (gc & 3)] = static_cast<uint8_t>(sb);
        }
    }
    __syncthreads();
    if constexpr (ROW) {
        if (tid < 64) {
            uint8_t* dst = R.scales + (rt * (R.kp >> 6) + ct * 2) * 512;
            reinterpret_cast<uint4*>(dst)[tid] = reinterpret_cast<const uint4*>(row_sc)[tid];
        }
    }
    if constexpr (COL) {
        // ---- phase B: a thread takes two adjacent source columns (one 32-bit shared load per source row) and
        //      encodes source rows g*16 .. g*16+15 of each ----
        const float inv_c = __fdiv_rn(1.f, __ldg(C.pts));
        const int cp = tid & 63;
        const bool c_rht = C.flags & NVFP4_Q_RHT, c_hi = C.flags & NVFP4_Q_HI_FIRST;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int g = (tid >> 6) + 4 * i;
            uint32_t w[16];
#pragma unroll
            for (int l = 0; l < 16; ++l) w[l] = *reinterpret_cast<const uint32_t*>(&tile[(g * 16 + l) * TILE_PITCH + 2 * cp]);
#pragma unroll
            for (int side = 0; side < 2; ++side) {
                const int n = 2 * cp + side;
                float v[16];
#pragma unroll
                for (int l = 0; l < 16; ++l) v[l] = __uint_as_float(side ? (w[l] & 0xffff0000u) : (w[l] << 16));
                if (c_rht) hadamard16_unscaled(v, sg);
                uint32_t sb;
                uint2 p = encode16<SR>(v, c_rht, inv_c, c_hi, C.seed + base, static_cast<uint64_t>(c0 + n) * C.kp + (r0 + g * 16), sb);
                *reinterpret_cast<uint2*>(col_out + n * COL_OUT_PITCH + g * 8) = p;
                col_sc[(g >> 2) * 512 + (n & 31) * 16 + (n >> 5) * 4 + (g & 3)] = static_cast<uint8_t>(sb);
            }
        }
        __syncthreads();
        if (tid < 64) {
            uint8_t* dst = C.scales + (ct * (C.kp >> 6) + rt * 2) * 512;
            reinterpret_cast<uint4*>(dst)[tid] = reinterpret_cast<const uint4*>(col_sc)[tid];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int ci = tid + 256 * i;
            const int nn = ci >> 3, ch = ci & 7;
            uint2 p = *reinterpret_cast<const uint2*>(col_out + nn * COL_OUT_PITCH + ch * 8);
            *reinterpret_cast<uint2*>(C.packed + (c0 + nn) * (C.kp >> 1) + (r0 >> 1) + ch * 8) = p;
        }
    }
}

template <int DT, int SR>
static void launch_tile_sr(const void* x, int64_t rows, int64_t cols, int64_t rs, int64_t cs, int vec_ok, const float* signs,
                           const int32_t* base, const Orient& R, const Orient& C, bool row, bool col, cudaStream_t st) {
    dim3 grid(static_cast<unsigned>(round128(rows) / 128), static_cast<unsigned>(round128(cols) / 128));
    if (row && col) quant_tile_kernel<DT, true, true, SR><<<grid, 256, 0, st>>>(x, rows, cols, rs, cs, vec_ok, signs, base, R, C);
    else if (row) quant_tile_kernel<DT, true, false, SR><<<grid, 256, 0, st>>>(x, rows, cols, rs, cs, vec_ok, signs, base, R, C);
    else quant_tile_kernel<DT, false, true, SR><<<grid, 256, 0, st>>>(x, rows, cols, rs, cs, vec_ok, signs, base, R, C);
}

template <int DT>
static int launch_tile(const void* x, int64_t rows, int64_t cols, int64_t rs, int64_t cs, int vec_ok,
                       const float* signs, const int32_t* base, const Orient& R, const Orient& C, bool row, bool col,
                       cudaStream_t st) {
    const int sr = sr_of_flags(row ? R.flags : C.flags);
    if (sr == SR_NONE) launch_tile_sr<DT, SR_NONE>(x, rows, cols, rs, cs, vec_ok, signs, base, R, C, row, col, st);
    else if (sr == SR_HASH) launch_tile_sr<DT, SR_HASH>(x, rows, cols, rs, cs, vec_ok, signs, base, R, C, row, col, st);
    else launch_tile_sr<DT, SR_PHILOX>(x, rows, cols, rs, cs, vec_ok, signs, base, R, C, row, col, st);
    return launch_status("nvfp4_quantize_tile");
}

// ================================================================================================
// dequantiser: one thread per 16-element group
// ================================================================================================
template <bool OUT_BF16>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ packed,
                                                      const uint8_t* __restrict__ scales,
                                                      const float* __restrict__ pts, int64_t kp, int64_t rows,
                                                      int64_t cols, int hi_first, void* __restrict__ out,
                                                      int64_t out_stride, int vec_ok) {
    const int64_t gpr = (cols + 15) >> 4;
    const int64_t gi = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gi >= rows * gpr) return;
    const int64_t r = gi / gpr, g = gi - r * gpr;
    const uint2 p = __ldg(reinterpret_cast<const uint2*>(packed + r * (kp >> 1) + g * 8));
    const float s = e4m3_to_float(__ldg(scales + scale_offset(r, g, kp >> 4)));
    const float t = __ldg(pts);
    const uint32_t w[2] = {p.x, p.y};
    float v[16];
#pragma unroll
    for (int l = 0; l < 16; ++l) {
        const uint32_t byte = (w[l >> 3] >> (8 * ((l >> 1) & 3))) & 0xffu;
        const uint32_t code = ((l & 1) ^ (hi_first ? 1 : 0)) ? (byte >> 4) : (byte & 15u);
        v[l] = __fmul_rn(__fmul_rn(e2m1_to_float(code), s), t);
    }
    const int64_t c0 = g * 16;
    if (vec_ok && c0 + 16 <= cols) {
        if constexpr (OUT_BF16) {
            uint32_t h[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) h[j] = bf16_bits(v[2 * j]) | (static_cast<uint32_t>(bf16_bits(v[2 * j + 1])) << 16);
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(out) + r * out_stride + c0);
            dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
            dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
        } else {
            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(out) + r * out_stride + c0);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
        return;
    }
#pragma unroll
    for (int l = 0; l < 16; ++l) {
        if (c0 + l < cols) {
            if constexpr (OUT_BF16) static_cast<__nv_bfloat16*>(out)[r * out_stride + c0 + l] = __float2bfloat16_rn(v[l]);
            else static_cast<float*>(out)[r * out_stride + c0 + l] = v[l];
        }
    }
}

}  // namespace nvfp4

// ================================================================================================
// C ABI
// ================================================================================================
using namespace nvfp4;

extern "C" const char* nvfp4_last_error(void) { return g_error; }
extern "C" int nvfp4_version(void) { return 1; }
extern "C" int64_t nvfp4_amax_scratch_bytes(void) { static_assert(sizeof(AmaxScratch) == SCRATCH_AMAX_OUT_OFFSET, "scratch layout");
    return SCRATCH_BYTES; }

static bool dtype_ok(int dt) { return dt == NVFP4_F32 || dt == NVFP4_BF16 || dt == NVFP4_F16; }

static int launch_amax(const void* x, int dtype, int64_t rows, int64_t cols, int64_t rs, int64_t cs, void* scratch,
                       float* out4, float* pts_dst, int which, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(x && scratch && out4, NVFP4_ERR_ARG, "nvfp4_amax: null pointer");
    NVFP4_REQUIRE(rows > 0 && cols > 0 && rs >= 0 && cs >= 0, NVFP4_ERR_ARG,
                  "nvfp4_amax: empty tensor or negative stride (rows=%lld cols=%lld)", (long long)rows, (long long)cols);
    NVFP4_REQUIRE(dtype_ok(dtype), NVFP4_ERR_DTYPE, "nvfp4_amax: unsupported dtype code %d", dtype);
    NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_amax: scratch must be 16-byte aligned");
    const int esz = dtype == NVFP4_F32 ? 4 : 2;
    const bool dense = (cs == 1 && rs == cols) || (rs == 1 && cs == rows) || (rows == 1 && cs == 1) || (cols == 1 && rs == 1);
    const int dense_vec = dense && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    const int64_t n = rows * cols;
    const int64_t per_block = static_cast<int64_t>(AMAX_THREADS) * (16 / esz) * 4;
    int blocks = static_cast<int>(std::min<int64_t>((n + per_block - 1) / per_block, AMAX_MAX_BLOCKS));
    blocks = std::max(blocks, 1);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    auto* sc = static_cast<AmaxScratch*>(scratch);
    if (dtype == NVFP4_F32) amax_kernel<NVFP4_F32><<<blocks, AMAX_THREADS, 0, st>>>(x, rows, cols, rs, cs, dense_vec, sc, out4, pts_dst, which);
    else if (dtype == NVFP4_BF16) amax_kernel<NVFP4_BF16><<<blocks, AMAX_THREADS, 0, st>>>(x, rows, cols, rs, cs, dense_vec, sc, out4, pts_dst, which);
    else amax_kernel<NVFP4_F16><<<blocks, AMAX_THREADS, 0, st>>>(x, rows, cols, rs, cs, dense_vec, sc, out4, pts_dst, which);
    return launch_status("nvfp4_amax");
}

extern "C" int nvfp4_amax(const void* x, int dtype, int64_t rows, int64_t cols, int64_t rs, int64_t cs, void* scratch,
                          float* out4, nvfp4_stream_t stream) {
    return launch_amax(x, dtype, rows, cols, rs, cs, scratch, out4, nullptr, 0, stream);
}

extern "C" int nvfp4_quantize_tile(const void* x, int dtype, int64_t rows, int64_t cols, int64_t rs, int64_t cs,
                                   const float* signs, const int32_t* seed_base, uint8_t* row_packed,
                                   uint8_t* row_scales, const float* row_pts, int row_flags, uint32_t row_seed,
                                   uint8_t* col_packed, uint8_t* col_scales, const float* col_pts, int col_flags,
                                   uint32_t col_seed, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(x && signs, NVFP4_ERR_ARG, "nvfp4_quantize_tile: null source or signs");
    NVFP4_REQUIRE(rows > 0 && cols > 0 && rs >= 0 && cs >= 0, NVFP4_ERR_ARG,
                  "nvfp4_quantize_tile: empty tensor or negative stride (rows=%lld cols=%lld)", (long long)rows, (long long)cols);
    NVFP4_REQUIRE(dtype_ok(dtype), NVFP4_ERR_DTYPE, "nvfp4_quantize_tile: unsupported dtype code %d", dtype);
    const bool row = row_packed != nullptr, col = col_packed != nullptr;
    NVFP4_REQUIRE(row || col, NVFP4_ERR_ARG, "nvfp4_quantize_tile: no output orientation requested");
    NVFP4_REQUIRE(!row || (row_scales && row_pts), NVFP4_ERR_ARG, "nvfp4_quantize_tile: row orientation needs scales and pts");
    NVFP4_REQUIRE(!col || (col_scales && col_pts), NVFP4_ERR_ARG, "nvfp4_quantize_tile: col orientation needs scales and pts");
    const int both_sr = NVFP4_Q_SR_HASH | NVFP4_Q_SR_PHILOX;
    NVFP4_REQUIRE((row_flags & both_sr) != both_sr && (col_flags & both_sr) != both_sr, NVFP4_ERR_ARG,
                  "nvfp4_quantize_tile: choose one stochastic rounding source");
    NVFP4_REQUIRE(!(row && col) || sr_of_flags(row_flags) == sr_of_flags(col_flags), NVFP4_ERR_ARG,
                  "nvfp4_quantize_tile: both orientations must use the same rounding source");
    const int64_t rp = round128(rows), cp = round128(cols);
    NVFP4_REQUIRE(cp / 128 <= 65535, NVFP4_ERR_ARG, "nvfp4_quantize_tile: more than 65535 column tiles");
    NVFP4_REQUIRE(rp / 128 <= 0x7fffffffLL, NVFP4_ERR_ARG, "nvfp4_quantize_tile: too many row tiles");
    for (const void* p : {static_cast<const void*>(row_packed), static_cast<const void*>(row_scales),
                          static_cast<const void*>(col_packed), static_cast<const void*>(col_scales)})
        NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_quantize_tile: outputs must be 16-byte aligned");
    const int esz = dtype == NVFP4_F32 ? 4 : 2;
    const int vec_ok = cs == 1 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (rs * esz) % 16 == 0;
    Orient R{row_packed, row_scales, row_pts, cp, row_seed, row_flags};
    Orient C{col_packed, col_scales, col_pts, rp, col_seed, col_flags};
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == NVFP4_F32) return launch_tile<NVFP4_F32>(x, rows, cols, rs, cs, vec_ok, signs, seed_base, R, C, row, col, st);
    if (dtype == NVFP4_BF16) return launch_tile<NVFP4_BF16>(x, rows, cols, rs, cs, vec_ok, signs, seed_base, R, C, row, col, st);
    return launch_tile<NVFP4_F16>(x, rows, cols, rs, cs, vec_ok, signs, seed_base, R, C, row, col, st);
}

extern "C" int nvfp4_quantize(const void* x, int dtype, int64_t m, int64_t k, int64_t s0, int64_t s1, int64_t mp,
                              int64_t kp, int sr, int rht, uint32_t seed, const float* signs, const float* given_scale,
                              const int32_t* seed_base, int pair, uint8_t* packed, uint8_t* scales, float* pts_out,
                              uint8_t* packed_t, uint8_t* scales_t, void* scratch, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(x && packed && scales && signs, NVFP4_ERR_ARG, "nvfp4_quantize: null pointer");
    NVFP4_REQUIRE(m > 0 && k > 0 && s0 >= 0 && s1 >= 0, NVFP4_ERR_ARG, "nvfp4_quantize: empty/broadcast/negative strides unsupported");
    NVFP4_REQUIRE(mp == round128(m) && kp == round128(k), NVFP4_ERR_ARG,
                  "nvfp4_quantize: padded dimensions must be the sizes rounded up to a multiple of 128");
    NVFP4_REQUIRE(sr == 0 || sr == NVFP4_Q_SR_HASH || sr == NVFP4_Q_SR_PHILOX, NVFP4_ERR_ARG, "nvfp4_quantize: bad sr mode %d", sr);
    NVFP4_REQUIRE(given_scale || (pts_out && scratch), NVFP4_ERR_ARG, "nvfp4_quantize: need pts_out and scratch when no scale is given");
    const float* pts = given_scale;
    if (!given_scale) {
        // the four amax results land in the scratch tail; the scale this call needs also goes to pts_out
        float* out4 = reinterpret_cast<float*>(static_cast<char*>(scratch) + SCRATCH_AMAX_OUT_OFFSET);
        int rc = launch_amax(x, dtype, m, k, s0, s1, scratch, out4, pts_out, rht ? 2 : 1, stream);
        if (rc != NVFP4_OK) return rc;
        pts = pts_out;
    }
    const int flags = (rht ? NVFP4_Q_RHT : 0) | sr;
    if (pair) {
        NVFP4_REQUIRE(!sr && !rht && s1 == 1 && s0 == k && packed_t && scales_t, NVFP4_ERR_ARG,
                      "nvfp4_quantize: paired encoding requires contiguous RNE weights and both outputs");
        return nvfp4_quantize_tile(x, dtype, m, k, s0, s1, signs, seed_base, packed, scales, pts, 0, 0, packed_t, scales_t, pts, 0, 0, stream);
    }
    if (s0 == 1 && s1 != 1) {
        // a transposed view of a row-major k x m matrix: its packing is the column orientation of that matrix
        return nvfp4_quantize_tile(x, dtype, k, m, s1, s0, signs, seed_base, nullptr, nullptr, nullptr, 0, 0, packed, scales, pts,
                                   flags, seed, stream);
    }
    return nvfp4_quantize_tile(x, dtype, m, k, s0, s1, signs, seed_base, packed, scales, pts, flags, seed, nullptr, nullptr, nullptr,
                               0, 0, stream);
}

extern "C" int nvfp4_dequantize(const uint8_t* packed, const uint8_t* scales, const float* pts, int64_t kp, int64_t rows,
                                int64_t cols, int hi_first, int out_dtype, void* out, int64_t out_stride,
                                nvfp4_stream_t stream) {
    NVFP4_REQUIRE(packed && scales && pts && out, NVFP4_ERR_ARG, "nvfp4_dequantize: null pointer");
    NVFP4_REQUIRE(rows > 0 && cols > 0 && kp % 128 == 0 && cols <= kp && out_stride >= cols, NVFP4_ERR_ARG,
                  "nvfp4_dequantize: bad shape (rows=%lld cols=%lld kp=%lld)", (long long)rows, (long long)cols, (long long)kp);
    NVFP4_REQUIRE(out_dtype == NVFP4_F32 || out_dtype == NVFP4_BF16, NVFP4_ERR_DTYPE, "nvfp4_dequantize: output must be FP32 or BF16");
    NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 7) == 0, NVFP4_ERR_ALIGN, "nvfp4_dequantize: payload must be 8-byte aligned");
    const int64_t groups = rows * ((cols + 15) / 16);
    const unsigned blocks = static_cast<unsigned>((groups + 255) / 256);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int esz = out_dtype == NVFP4_BF16 ? 2 : 4;
    const int vec_ok = (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (out_stride * esz) % 16 == 0;
    if (out_dtype == NVFP4_BF16) dequant_kernel<true><<<blocks, 256, 0, st>>>(packed, scales, pts, kp, rows, cols, hi_first, out, out_stride, vec_ok);
    else dequant_kernel<false><<<blocks, 256, 0, st>>>(packed, scales, pts, kp, rows, cols, hi_first, out, out_stride, vec_ok);
    return launch_status("nvfp4_dequantize");
}

// ================================================================================================
// Entry point for callers that cannot allocate device memory
// ================================================================================================
namespace nvfp4 {
// Scratch of the amax stage for nvfp4_quantize_static: lives in the library image, one copy per GPU that loads it.
static __device__ __align__(256) unsigned char g_static_scratch[SCRATCH_BYTES];
constexpr int64_t STATIC_MAX_ELEMENTS = int64_t(1) << 31;
constexpr int MAX_DEVICES = 64;
static void* g_static_scratch_addr[MAX_DEVICES] = {};
}  // namespace nvfp4

extern "C" int64_t nvfp4_quantize_static_max_elements(void) { return STATIC_MAX_ELEMENTS; }

extern "C" int nvfp4_quantize_static(const void* x, int dtype, int64_t m, int64_t k, int64_t s0, int64_t s1, int64_t mp,
                                     int64_t kp, int sr, int rht, uint32_t seed, const float* signs, const int32_t* seed_base,
                                     uint8_t* packed, uint8_t* scales, float* pts_out, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(x && packed && scales && signs && pts_out, NVFP4_ERR_ARG, "nvfp4_quantize_static: null pointer");
    NVFP4_REQUIRE(m > 0 && k > 0, NVFP4_ERR_ARG, "nvfp4_quantize_static: empty tensor");
    NVFP4_REQUIRE(m <= STATIC_MAX_ELEMENTS / k, NVFP4_ERR_ARG,
                  "nvfp4_quantize_static: %lld x %lld elements exceed the limit of %lld of the built-in scratch variant; "
                  "use nvfp4_quantize with caller-provided scratch", (long long)m, (long long)k, (long long)STATIC_MAX_ELEMENTS);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    NVFP4_REQUIRE(e == cudaSuccess && dev >= 0 && dev < MAX_DEVICES, NVFP4_ERR_LAUNCH, "nvfp4_quantize_static: no usable current device");
    if (!g_static_scratch_addr[dev]) {
        // The symbol name is only a host-side handle; the kernel needs the address the array has on THIS device.
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_static_scratch);
        NVFP4_REQUIRE(e == cudaSuccess && addr, NVFP4_ERR_LAUNCH, "nvfp4_quantize_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_static_scratch_addr[dev] = addr;
    }
    void* scratch = g_static_scratch_addr[dev];
    // Every call shares the array and it keeps what the last call left: the arrival ticket must start at zero.
    e = cudaMemsetAsync(static_cast<char*>(scratch) + offsetof(AmaxScratch, ticket), 0, sizeof(unsigned int),
                        reinterpret_cast<cudaStream_t>(stream));
    NVFP4_REQUIRE(e == cudaSuccess, NVFP4_ERR_LAUNCH, "nvfp4_quantize_static: cannot clear the ticket: %s", cudaGetErrorString(e));
    return nvfp4_quantize(x, dtype, m, k, s0, s1, mp, kp, sr, rht, seed, signs, nullptr, seed_base, 0, packed, scales, pts_out,
                          nullptr, nullptr, scratch, stream);
}
