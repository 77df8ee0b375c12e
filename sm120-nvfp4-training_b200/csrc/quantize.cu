// NVFP4 quantiser for sm_100a: tensor amax, the two tile quantisers (row packing and/or transposed packing from one
// read of the source), dequantiser.  The group arithmetic and its numerical contract live in quant_core.cuh.
//
//   quant_stream_kernel  persistent: 128 x 128 source tiles stream into a shared-memory ring by TMA loads (out-of-range
//                        rows / columns arrive as zeros); eight warps encode from shared memory, each into its own staging
//                        slabs, which leave by TMA stores; the ring is refilled by the last warp to finish a stage or, in
//                        the hash mode, by a ninth warp.
//                        Serves 2-byte sources with unit column stride and 16-byte aligned rows.
//   quant_tile_kernel    one 128 x 128 tile per CTA with per-thread loads: every other source (FP32, E4M3 x unit,
//                        arbitrary strides, unaligned bases).
//   quant_resident_kernel  amax + row packing in one cooperative launch for BF16 tensors that fit the GPU's shared
//                        memory (one read of the source from HBM); used by the nvfp4_quantize operator.
#include "quant_core.cuh"
#include "async.cuh"

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
// tile quantiser: 128 x 128 source tile per CTA, 256 threads
// ================================================================================================
constexpr int TILE = 128;
constexpr int TILE_PITCH = TILE + 8;  // bf16 elements per smem row (272 B keeps 16-byte alignment)
constexpr int COL_OUT_PITCH = 72;     // bytes per transposed payload row in smem (64 + 8: conflict-free 8-byte stores)

// `unit` is read for E4M3 sources only: a contiguous weight whose element (r, c) is e4m3 * unit[(r * cols + c) / 512],
// rounded to BF16 like every other source.
template <int DT>
__device__ __forceinline__ void load_group_bf16(const void* x, int64_t r, int64_t c0, int64_t rows, int64_t cols,
                                                int64_t rs, int64_t cs, bool vec_ok, const float* unit, uint16_t (&h)[16]) {
    if (r >= rows || c0 >= cols) {
#pragma unroll
        for (int l = 0; l < 16; ++l) h[l] = 0;
        return;
    }
    if constexpr (DT == NVFP4_E4M3) {
        const uint8_t* src = static_cast<const uint8_t*>(x);
        const int64_t flat = r * cols + c0;
        if (vec_ok && c0 + 16 <= cols) {   // 16 codes in one 16-byte load; cols % 16 == 0, so they share a unit
            const uint4 u = __ldg(reinterpret_cast<const uint4*>(src + flat));
            const float scale = __ldg(unit + (flat >> 9));
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int l = 0; l < 16; ++l) h[l] = bf16_bits(__fmul_rn(e4m3_to_float((w[l >> 2] >> (8 * (l & 3))) & 255u), scale));
            return;
        }
#pragma unroll
        for (int l = 0; l < 16; ++l)
            h[l] = (c0 + l < cols) ? bf16_bits(__fmul_rn(e4m3_to_float(src[flat + l]), __ldg(unit + ((flat + l) >> 9)))) : uint16_t(0);
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
    if constexpr (DT != NVFP4_E4M3) {
#pragma unroll
        for (int l = 0; l < 16; ++l) h[l] = (c0 + l < cols) ? load_as_bf16<DT>(x, r * rs + (c0 + l) * cs) : uint16_t(0);
    }
}

template <int DT, bool ROW, bool COL, int SR>
__global__ void __launch_bounds__(256, 4) quant_tile_kernel(const void* __restrict__ x, int64_t rows, int64_t cols,
                                                         int64_t rs, int64_t cs, int vec_ok,
                                                         const float* __restrict__ signs,
                                                         const int32_t* __restrict__ seed_base,
                                                         const float* __restrict__ unit, const float* __restrict__ amax,
                                                         Orient R, Orient C) {
    __shared__ __align__(16) uint16_t tile[COL ? TILE * TILE_PITCH : 8];
    __shared__ __align__(16) uint8_t row_sc[ROW ? 1024 : 16];
    __shared__ __align__(16) uint8_t col_sc[COL ? 1024 : 16];
    __shared__ __align__(16) uint8_t col_out[COL ? TILE * COL_OUT_PITCH : 16];

    const int tid = threadIdx.x;
    const int64_t rt = blockIdx.x, ct = blockIdx.y;
    const int64_t r0 = rt * TILE, c0 = ct * TILE;
    float sg[16];
#pragma unroll
    for (int l = 0; l < 16; ++l) sg[l] = signs ? __ldg(signs + l) : 1.f;   // null: no orientation uses the transform
    const uint32_t base = seed_base ? static_cast<uint32_t>(__ldg(seed_base)) : 0u;

    const bool writer = tid == 0 && blockIdx.x == 0 && blockIdx.y == 0;
    ScaleMath sm_r{0.f, false};
    if constexpr (ROW) sm_r = scale_math(tensor_scale(amax, R.pts, R.flags & NVFP4_Q_RHT, writer));

    // ---- phase A: each thread owns 4 row groups (16 consecutive columns of one row) ----------------
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gi = tid + 256 * i;
        const int lr = gi >> 3, gc = gi & 7;
        const int64_t r = r0 + lr, c = c0 + gc * 16;
        uint16_t h[16];
        load_group_bf16<DT>(x, r, c, rows, cols, rs, cs, vec_ok != 0, unit, h);
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
            const uint64_t idx0 = static_cast<uint64_t>(r) * R.kp + c;
            uint2 p = encode16<SR, false>(v, rht, sm_r.inv, R.seed + base, static_cast<uint32_t>(idx0), idx0 >> 4, sb);
            if (R.flags & NVFP4_Q_HI_FIRST) p = swap_nibbles(p);
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
        const ScaleMath sm_c = scale_math(tensor_scale(amax, C.pts, C.flags & NVFP4_Q_RHT, writer));
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
                const uint64_t idx0 = static_cast<uint64_t>(c0 + n) * C.kp + (r0 + g * 16);
                uint2 p = encode16<SR, false>(v, c_rht, sm_c.inv, C.seed + base, static_cast<uint32_t>(idx0), idx0 >> 4, sb);
                if (c_hi) p = swap_nibbles(p);
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
                           const int32_t* base, const float* unit, const float* amax, const Orient& R, const Orient& C, bool row,
                           bool col, cudaStream_t st) {
    dim3 grid(static_cast<unsigned>(round128(rows) / 128), static_cast<unsigned>(round128(cols) / 128));
    if (row && col) quant_tile_kernel<DT, true, true, SR><<<grid, 256, 0, st>>>(x, rows, cols, rs, cs, vec_ok, signs, base, unit, amax, R, C);
    else if (row) quant_tile_kernel<DT, true, false, SR><<<grid, 256, 0, st>>>(x, rows, cols, rs, cs, vec_ok, signs, base, unit, amax, R, C);
    else quant_tile_kernel<DT, false, true, SR><<<grid, 256, 0, st>>>(x, rows, cols, rs, cs, vec_ok, signs, base, unit, amax, R, C);
}

template <int DT>
static int launch_tile(const void* x, int64_t rows, int64_t cols, int64_t rs, int64_t cs, int vec_ok, const float* signs,
                       const int32_t* base, const float* unit, const float* amax, const Orient& R, const Orient& C, bool row,
                       bool col, cudaStream_t st) {
    const int sr = sr_of_flags(row ? R.flags : C.flags);
    if (sr == SR_NONE) launch_tile_sr<DT, SR_NONE>(x, rows, cols, rs, cs, vec_ok, signs, base, unit, amax, R, C, row, col, st);
    else if constexpr (DT == NVFP4_E4M3) return NVFP4_ERR_UNSUPPORTED;   // master weights are rounded to nearest
    else if (sr == SR_HASH) launch_tile_sr<DT, SR_HASH>(x, rows, cols, rs, cs, vec_ok, signs, base, unit, amax, R, C, row, col, st);
    else launch_tile_sr<DT, SR_PHILOX>(x, rows, cols, rs, cs, vec_ok, signs, base, unit, amax, R, C, row, col, st);
    return launch_status("nvfp4_quantize_tile");
}

// ================================================================================================
// streaming quantiser: persistent CTAs, TMA tile loads into a shared-memory ring, TMA / bulk stores
// ================================================================================================
constexpr int QS_STAGES = 2;            // source tiles in flight per CTA (two CTAs per SM: four per SM, 128 KB)
constexpr int QS_COMPUTE_WARPS = 8;
// Two ways to keep the ring full.  LOADER: a ninth warp waits for a stage's `empty` barrier and issues the next load (288
// threads, 96 registers per thread).  Without it the last encoding warp to finish with a stage issues the load itself (256
// threads, which leaves 128 registers per thread: no spills).  Measured on both packings of 8192 x 4096: Philox 40.0 -> 36.9
// us without the loader, the reference's hash generator 97.9 -> 110 us; round to nearest the same.  So hash keeps the loader.
__host__ __device__ constexpr bool qs_loader(int sr) { return sr == SR_HASH; }
__host__ __device__ constexpr int qs_threads(int sr) { return QS_COMPUTE_WARPS * 32 + (qs_loader(sr) ? 32 : 0); }
constexpr int QS_TILE_BYTES = TILE * TILE * 2;
constexpr int QS_SLAB = TILE / QS_COMPUTE_WARPS;          // 16 packing rows per warp and orientation

// What one encoding warp owns: two sets of payload slabs (16 rows of 64 bytes per orientation; a store may still be
// reading one set while the next tile is written into the other) and the scale bytes of the current tile.
struct __align__(128) WarpStage {
    uint8_t row_out[2][QS_SLAB * 64];
    uint8_t col_out[2][QS_SLAB * 64];
    uint8_t row_sc[QS_SLAB * 8];
    uint8_t col_sc[QS_SLAB * 8];
};

// TR = source rows per tile: 128, or 64 for kernels that produce the row orientation only (twice the tiles, which evens
// out the tiles per CTA of tensors with few of them); the ring holds 64 KB either way.
template <int TR>
struct __align__(128) StreamSmem {
    static constexpr int STAGES = QS_STAGES * TILE / TR;
    uint16_t in[STAGES][TR * TILE];        // dense rows of 256 bytes, as the tile load writes them
    WarpStage stage[QS_COMPUTE_WARPS];
    uint64_t full[STAGES];
    uint64_t empty[STAGES];                // LOADER: the eight warps have finished reading the stage's tile
    unsigned int released[STAGES];         // without LOADER: count of warps that have finished with it
    int abort;
};

struct StreamArgs {
    const float* signs;
    const float* amax;    // nullable: tensor amax left on the device by the producer of the source
    const int32_t* seed_base;
    int* status;          // nullable device int, raised when a bounded wait gave up
    Orient R, C;
    int tiles_r, tiles_c;   // tiles of TR x 128 source elements
};

template <int DT>
__device__ __forceinline__ void unpack16(const uint4 a, const uint4 b, float (&v)[16]) {
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        if constexpr (DT == NVFP4_BF16) {
            v[2 * t] = __uint_as_float(w[t] << 16);
            v[2 * t + 1] = __uint_as_float(w[t] & 0xffff0000u);
        } else {   // FP16 -> FP32 is exact, then the one rounding to BF16 every source goes through
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
            v[2 * t] = bf16_value(bf16_bits(f.x));
            v[2 * t + 1] = bf16_value(bf16_bits(f.y));
        }
    }
}

// The tile loop of one encoding warp.  FAST selects the division-free scale arithmetic; it is decided once per launch from
// the tensor scales, so no group pays for a branch.
template <int DT, bool ROW, bool COL, int SR, bool R_RHT, bool C_RHT, bool FAST, int TR>
__device__ __forceinline__ void stream_encode_loop(StreamSmem<TR>& S, const CUtensorMap* map_in, const CUtensorMap* map_row, const CUtensorMap* map_col,
                                                   const StreamArgs& a, const float (&sg)[16], float inv_r, float inv_c,
                                                   int warp, int lane) {
    using namespace aop;
    const uint32_t base = a.seed_base ? static_cast<uint32_t>(__ldg(a.seed_base)) : 0u;
    const uint32_t seed_r = a.R.seed + base, seed_c = a.C.seed + base;
    static_assert(TR == TILE || !COL, "the transposed orientation needs square tiles");
    constexpr int STAGES = StreamSmem<TR>::STAGES;
    constexpr int SLAB = TR / QS_COMPUTE_WARPS;   // packing rows of the row orientation per warp: 16 or 8
    WarpStage& W = S.stage[warp];
    const int slab = warp * SLAB;             // first source row of this warp inside a tile
    const int slab_c = warp * QS_SLAB;        // first source column of this warp inside a tile (transposed orientation)
    const int piece_half = lane & 1;          // the 4-byte scale pieces this lane stores: row slab + lane / 2, half lane % 2
    const int64_t gpr_r = a.R.kp >> 4, gpr_c = a.C.kp >> 4;            // groups per packing row
    const int n_tiles = a.tiles_r * a.tiles_c;
    int it = 0;
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++it) {
        const int s = it % STAGES, buf = it & 1;
        const int rt = t / a.tiles_c, ct = t - rt * a.tiles_c;
        // the stores issued two tiles ago have finished reading the staging set that is written next
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
        if (!__all_sync(0xffffffffu, mbar_wait(&S.full[s], (it / STAGES) & 1, &S.abort))) break;
        const uint16_t* tile = S.in[s];
        if constexpr (ROW) {
            // SLAB source rows x 8 groups: a lane owns SLAB / 4 groups; the warp reads 1 KB of consecutive bytes at a time
            const uint64_t group0 = static_cast<uint64_t>(rt * TR + slab) * gpr_r + ct * 8;
            // all of the lane's loads are issued before the first one is used
            uint4 raw[SLAB / 4][2];
#pragma unroll
            for (int i = 0; i < SLAB / 4; ++i) {
                const uint4* src = reinterpret_cast<const uint4*>(tile + (slab + 4 * i + (lane >> 3)) * TILE + (lane & 7) * 16);
                raw[i][0] = src[0]; raw[i][1] = src[1];
            }
#pragma unroll
            for (int i = 0; i < SLAB / 4; ++i) {
                const int lr = 4 * i + (lane >> 3), gc = lane & 7;
                float v[16];
                unpack16<DT>(raw[i][0], raw[i][1], v);
                if constexpr (R_RHT) hadamard16_unscaled(v, sg);
                const uint64_t group = group0 + static_cast<uint32_t>(lr * static_cast<int>(gpr_r) + gc);
                uint32_t sb;
                const uint2 p = encode16<SR, FAST>(v, R_RHT, inv_r, seed_r, static_cast<uint32_t>(group) << 4, group, sb);
                *reinterpret_cast<uint2*>(&W.row_out[buf][lr * 64 + gc * 8]) = p;
                W.row_sc[lr * 8 + gc] = static_cast<uint8_t>(sb);
            }
        }
        if constexpr (COL) {
            // 16 source columns x 8 groups of 16 source rows: a lane takes a pair of adjacent columns (one 32-bit shared
            // load per source row) for two groups
            const int cpl = lane & 7;
            const uint64_t group0 = static_cast<uint64_t>(ct * TILE + slab_c) * gpr_c + rt * 8;
            uint32_t wall[2][16];   // both groups' loads are issued before the first one is used
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int l = 0; l < 16; ++l)
                    wall[i][l] = *reinterpret_cast<const uint32_t*>(tile + (((lane >> 3) + 4 * i) * 16 + l) * TILE + slab_c + 2 * cpl);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int g = (lane >> 3) + 4 * i;
                const uint32_t (&w)[16] = wall[i];
#pragma unroll
                for (int side = 0; side < 2; ++side) {
                    const int n = 2 * cpl + side;
                    float v[16];
#pragma unroll
                    for (int l = 0; l < 16; ++l) {
                        if constexpr (DT == NVFP4_BF16) v[l] = __uint_as_float(side ? (w[l] & 0xffff0000u) : (w[l] << 16));
                        else {
                            const __half hv = __ushort_as_half(static_cast<unsigned short>(side ? (w[l] >> 16) : (w[l] & 0xffffu)));
                            v[l] = bf16_value(bf16_bits(__half2float(hv)));
                        }
                    }
                    if constexpr (C_RHT) hadamard16_unscaled(v, sg);
                    const uint64_t group = group0 + static_cast<uint32_t>(n * static_cast<int>(gpr_c) + g);
                    uint32_t sb;
                    const uint2 p = encode16<SR, FAST>(v, C_RHT, inv_c, seed_c, static_cast<uint32_t>(group) << 4, group, sb);
                    *reinterpret_cast<uint2*>(&W.col_out[buf][n * 64 + g * 8]) = p;
                    W.col_sc[n * 8 + g] = static_cast<uint8_t>(sb);
                }
            }
        }
        // this warp has read everything it needs from the source tile; its staging writes become visible to the copy
        // engine and to the lanes that store the scale pieces
        fence_async_shared();
        __syncwarp();
        if constexpr (qs_loader(SR)) {
            if (lane == 0) mbar_arrive(&S.empty[s]);
        } else if (lane == 0) {
            // the last of the eight warps to finish with this stage loads the tile that will use it next
            if (atomicAdd(&S.released[s], 1u) == QS_COMPUTE_WARPS - 1) {
                atomicExch(&S.released[s], 0u);
                const int next = t + STAGES * static_cast<int>(gridDim.x);
                if (next < n_tiles) {
                    const int nrt = next / a.tiles_c, nct = next - nrt * a.tiles_c;
                    fence_async_shared();
                    mbar_expect_tx(&S.full[s], TR * TILE * 2);
                    tma_load_2d(S.in[s], map_in, nct * TILE, nrt * TR, &S.full[s]);
                }
            }
        }
        if constexpr (ROW) {
            if (SLAB == QS_SLAB || lane < 2 * SLAB) {
                const int prow = rt * TR + slab + (lane >> 1);     // packing row of this piece; 128 of them share a block
                const uint32_t piece = *reinterpret_cast<const uint32_t*>(&W.row_sc[(lane >> 1) * 8 + piece_half * 4]);
                *reinterpret_cast<uint32_t*>(a.R.scales + (static_cast<int64_t>(prow >> 7) * (a.R.kp >> 6) + ct * 2 + piece_half) * 512 +
                                             (prow & 31) * 16 + ((prow & 127) >> 5) * 4) = piece;
            }
        }
        if constexpr (COL) {
            const int prow = slab_c + (lane >> 1);
            const uint32_t piece = *reinterpret_cast<const uint32_t*>(&W.col_sc[(lane >> 1) * 8 + piece_half * 4]);
            *reinterpret_cast<uint32_t*>(a.C.scales + (static_cast<int64_t>(ct) * (a.C.kp >> 6) + rt * 2 + piece_half) * 512 +
                                         (prow & 31) * 16 + (prow >> 5) * 4) = piece;
        }
        if (lane == 0) {
            if constexpr (ROW) tma_store_2d(map_row, ct * 64, rt * TR + slab, W.row_out[buf]);
            if constexpr (COL) tma_store_2d(map_col, rt * 64, ct * TILE + slab_c, W.col_out[buf]);
            bulk_commit();
        }
        __syncwarp();   // the scale bytes have been read before the next tile overwrites them
    }
    if (lane == 0) bulk_wait_all();
}

// Every encoding warp works on its own: of each 128 x 128 source tile it takes packing rows 16w .. 16w+15 of the row
// orientation (source rows) and of the transposed orientation (source columns), stages the 1 KB payload slabs in its own
// shared memory, hands them to the copy engine (one TMA store per slab) and writes its scale bytes as 4-byte pieces of the
// swizzled blocks.  The only block-wide events are the ring's full barriers and the per-stage release counters.
template <int DT, bool ROW, bool COL, int SR, bool R_RHT, bool C_RHT, int TR>
__device__ __forceinline__ void quant_stream_body(const CUtensorMap& map_in, const CUtensorMap& map_row, const CUtensorMap& map_col,
                                                  const StreamArgs& a) {
    using namespace aop;
    using Smem = StreamSmem<TR>;
    extern __shared__ __align__(128) uint8_t stream_smem_raw[];
    Smem& S = *reinterpret_cast<Smem*>(stream_smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_tiles = a.tiles_r * a.tiles_c;
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < Smem::STAGES; ++s) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], QS_COMPUTE_WARPS); S.released[s] = 0u; }
        S.abort = 0;
        fence_barrier_init();
        if constexpr (!qs_loader(SR)) {
            // the first tiles of this CTA; later ones are requested by the warp that frees a stage
            for (int s = 0; s < Smem::STAGES; ++s) {
                const int t = blockIdx.x + s * static_cast<int>(gridDim.x);
                if (t >= n_tiles) break;
                const int rt = t / a.tiles_c, ct = t - rt * a.tiles_c;
                mbar_expect_tx(&S.full[s], TR * TILE * 2);
                tma_load_2d(S.in[s], &map_in, ct * TILE, rt * TR, &S.full[s]);
            }
        }
    }
    __syncthreads();
    if (qs_loader(SR) && warp == QS_COMPUTE_WARPS) {
        // ---- loading warp: keeps the ring full --------------------------------------------------------------------
        int it = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++it) {
            const int s = it % Smem::STAGES;
            if (it >= Smem::STAGES) {
                const bool ok = mbar_wait(&S.empty[s], ((it / Smem::STAGES) - 1) & 1, &S.abort);
                if (!__all_sync(0xffffffffu, ok)) break;
            }
            if (elect_one()) {
                const int rt = t / a.tiles_c, ct = t - rt * a.tiles_c;
                mbar_expect_tx(&S.full[s], TR * TILE * 2);
                tma_load_2d(S.in[s], &map_in, ct * TILE, rt * TR, &S.full[s]);
            }
            __syncwarp();
        }
    } else {
        float sg[16];
#pragma unroll
        for (int l = 0; l < 16; ++l) sg[l] = a.signs ? __ldg(a.signs + l) : 1.f;
        ScaleMath sm_r{1.f, true}, sm_c{1.f, true};
        const bool writer = tid == 0 && blockIdx.x == 0;
        if constexpr (ROW) sm_r = scale_math(tensor_scale(a.amax, a.R.pts, R_RHT, writer));
        if constexpr (COL) sm_c = scale_math(tensor_scale(a.amax, a.C.pts, C_RHT, writer));
        if (sm_r.fast && sm_c.fast)
            stream_encode_loop<DT, ROW, COL, SR, R_RHT, C_RHT, true, TR>(S, &map_in, &map_row, &map_col, a, sg, sm_r.inv, sm_c.inv, warp, lane);
        else
            stream_encode_loop<DT, ROW, COL, SR, R_RHT, C_RHT, false, TR>(S, &map_in, &map_row, &map_col, a, sg, sm_r.inv, sm_c.inv, warp, lane);
    }
    __syncthreads();
    if (tid == 0 && S.abort && a.status) *a.status = NVFP4_ERR_TIMEOUT;
}

template <int DT, bool ROW, bool COL, int SR, bool R_RHT, bool C_RHT, int TR>
__global__ void __launch_bounds__(qs_threads(SR), 2)
quant_stream_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_row,
                    const __grid_constant__ CUtensorMap map_col, const StreamArgs a) {
    quant_stream_body<DT, ROW, COL, SR, R_RHT, C_RHT, TR>(map_in, map_row, map_col, a);
}

static bool stream_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("NVFP4_QUANT_STREAM");
        on = !(e && e[0] == '0');
    }
    return on != 0;
}

constexpr int QS_ROW_ONLY_TILE_ROWS = 128;   // 64-row tiles were measured: 13.2 us against 11.8 us per 4096 x 4096 tensor

template <int DT, bool ROW, bool COL, int SR, bool R_RHT, bool C_RHT>
static cudaError_t launch_stream_one(const CUtensorMap& mi, const CUtensorMap& mr, const CUtensorMap& mc, const StreamArgs& a,
                                     int grid, cudaStream_t st) {
    constexpr int TR = COL ? TILE : QS_ROW_ONLY_TILE_ROWS;
    const size_t smem = sizeof(StreamSmem<TR>);
    auto kernel = quant_stream_kernel<DT, ROW, COL, SR, R_RHT, C_RHT, TR>;
    static bool configured = false;   // one flag per kernel instantiation; the attribute belongs to the function
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        configured = true;
    }
    kernel<<<grid, qs_threads(SR), smem, st>>>(mi, mr, mc, a);
    return cudaSuccess;
}

// Orientation / transform combinations the streaming kernel is built for: one orientation with or without the Hadamard
// transform, both orientations without it (weights) or with it on the transposed one (activations, gradients).
template <int DT, int SR>
static cudaError_t launch_stream_sr(const CUtensorMap& mi, const CUtensorMap& mr, const CUtensorMap& mc, const StreamArgs& a,
                                    bool row, bool col, int grid, cudaStream_t st) {
    const bool rr = a.R.flags & NVFP4_Q_RHT, cr = a.C.flags & NVFP4_Q_RHT;
    if (row && col) {
        if (cr) return launch_stream_one<DT, true, true, SR, false, true>(mi, mr, mc, a, grid, st);
        return launch_stream_one<DT, true, true, SR, false, false>(mi, mr, mc, a, grid, st);
    }
    if (row) {
        if (rr) return launch_stream_one<DT, true, false, SR, true, false>(mi, mr, mc, a, grid, st);
        return launch_stream_one<DT, true, false, SR, false, false>(mi, mr, mc, a, grid, st);
    }
    if (cr) return launch_stream_one<DT, false, true, SR, false, true>(mi, mr, mc, a, grid, st);
    return launch_stream_one<DT, false, true, SR, false, false>(mi, mr, mc, a, grid, st);
}

// Returns NVFP4_ERR_UNSUPPORTED when the source does not qualify (the caller then uses the tile kernel).
static int try_stream(const void* x, int dtype, int64_t rows, int64_t cols, int64_t rs, int64_t cs, const float* signs,
                      const float* amax, const int32_t* base, int* status, const Orient& R, const Orient& C, bool row, bool col,
                      cudaStream_t st) {
    if (!stream_enabled() || (dtype != NVFP4_BF16 && dtype != NVFP4_F16) || cs != 1) return NVFP4_ERR_UNSUPPORTED;
    const int sr_mode = sr_of_flags(row ? R.flags : C.flags);
    if (dtype == NVFP4_F16 && sr_mode != SR_NONE) return NVFP4_ERR_UNSUPPORTED;          // FP16 sources are master weights
    if (((row ? R.flags : 0) | (col ? C.flags : 0)) & NVFP4_Q_HI_FIRST) return NVFP4_ERR_UNSUPPORTED;
    if (row && col && (R.flags & NVFP4_Q_RHT)) return NVFP4_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (rs * 2) % 16 != 0 || rs < cols) return NVFP4_ERR_UNSUPPORTED;
    const int64_t rp = round128(rows), cp = round128(cols);
    if (rp / 64 * (cp / 128) > 0x7fffffffLL || rp > 0x7fffffffLL || cp > 0x7fffffffLL) return NVFP4_ERR_UNSUPPORTED;
    const int tr = col ? TILE : QS_ROW_ONLY_TILE_ROWS;      // source rows per tile
    CUtensorMap mi, mr, mc;
    if (!aop::make_map_2d(&mi, dtype == NVFP4_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x,
                          static_cast<uint64_t>(cols), static_cast<uint64_t>(rows), static_cast<uint64_t>(rs) * 2, TILE, tr))
        return NVFP4_ERR_UNSUPPORTED;
    mr = mi; mc = mi;
    if (row && !aop::make_map_2d(&mr, CU_TENSOR_MAP_DATA_TYPE_UINT8, R.packed, static_cast<uint64_t>(cp / 2), static_cast<uint64_t>(rp),
                                 static_cast<uint64_t>(cp / 2), 64, tr / QS_COMPUTE_WARPS))
        return NVFP4_ERR_UNSUPPORTED;
    if (col && !aop::make_map_2d(&mc, CU_TENSOR_MAP_DATA_TYPE_UINT8, C.packed, static_cast<uint64_t>(rp / 2), static_cast<uint64_t>(cp),
                                 static_cast<uint64_t>(rp / 2), 64, QS_SLAB))
        return NVFP4_ERR_UNSUPPORTED;
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    StreamArgs a{signs, amax, base, status, R, C, static_cast<int>(rp / tr), static_cast<int>(cp / 128)};
    const int64_t tiles = static_cast<int64_t>(a.tiles_r) * a.tiles_c;
    const int grid = static_cast<int>(std::min<int64_t>(tiles, 2LL * sms));
    cudaError_t e;
    if (dtype == NVFP4_F16) e = launch_stream_sr<NVFP4_F16, SR_NONE>(mi, mr, mc, a, row, col, grid, st);
    else if (sr_mode == SR_NONE) e = launch_stream_sr<NVFP4_BF16, SR_NONE>(mi, mr, mc, a, row, col, grid, st);
    else if (sr_mode == SR_HASH) e = launch_stream_sr<NVFP4_BF16, SR_HASH>(mi, mr, mc, a, row, col, grid, st);
    else e = launch_stream_sr<NVFP4_BF16, SR_PHILOX>(mi, mr, mc, a, row, col, grid, st);
    if (e != cudaSuccess) {
        set_error("nvfp4_quantize_tile: cannot configure the streaming kernel: %s", cudaGetErrorString(e));
        return NVFP4_ERR_LAUNCH;
    }
    return launch_status("nvfp4_quantize_tile");
}

// ================================================================================================
// resident quantiser: tensor amax AND row packing in one launch, the source read from HBM once
// ================================================================================================
// A BF16 tensor of at most QR_MAX_TILES x (number of SMs) source tiles (33.9 MB on 148 SMs) fits the GPU's shared memory.
// One CTA per SM loads its tiles with TMA (all loads in flight at once), takes the magnitude maximum of what arrived,
// meets the other CTAs at a grid barrier (cooperative launch, bounded wait), derives the tensor scale from the global
// maximum with the amax kernel's expression, and encodes its tiles from shared memory.  A warp overwrites the 4 KB source
// slab it has just read into registers with the slab's 1 KB of payload, which leaves by a TMA store.
constexpr int QR_MAX_TILES = 7;
constexpr int QR_WARPS = 16;
constexpr int QR_THREADS = QR_WARPS * 32;

struct __align__(128) ResidentSmem {
    uint16_t in[QR_MAX_TILES][TILE * TILE];
    uint64_t full[QR_MAX_TILES];
    uint32_t warp_best[QR_WARPS];
    uint32_t amax_bits;
    int proceed;
    int abort;
};

struct ResidentArgs {
    const float* signs;
    const int32_t* seed_base;
    unsigned int* amax_word;   // zero between launches: maximum of the magnitude bits over all CTAs
    unsigned int* arrivals;    // zero between launches: grid barrier
    float* out4;               // the four results of the amax kernel
    int* status;
    Orient R;
    int tiles_r, tiles_c;
};

template <int SR, bool R_RHT, bool FAST>
__device__ __forceinline__ void resident_encode(ResidentSmem& S, const CUtensorMap* map_row, const ResidentArgs& a,
                                                const float (&sg)[16], float inv, int my_tiles, int warp, int lane) {
    using namespace aop;
    const uint32_t seed = a.R.seed + (a.seed_base ? static_cast<uint32_t>(__ldg(a.seed_base)) : 0u);
    const int64_t gpr = a.R.kp >> 4;
    for (int item = warp; item < my_tiles * 8; item += QR_WARPS) {
        const int k = item >> 3, slab = (item & 7) * QS_SLAB;
        const int t = blockIdx.x + k * gridDim.x;
        const int rt = t / a.tiles_c, ct = t - rt * a.tiles_c;
        uint16_t* rows16 = S.in[k] + slab * TILE;       // this warp's 16 source rows of 256 bytes
        uint4 raw[4][2];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4* src = reinterpret_cast<const uint4*>(rows16 + (4 * i + (lane >> 3)) * TILE + (lane & 7) * 16);
            raw[i][0] = src[0]; raw[i][1] = src[1];
        }
        __syncwarp();                                   // the whole slab is in registers: its memory becomes the staging area
        uint8_t* out = reinterpret_cast<uint8_t*>(rows16);
        uint8_t* out_sc = out + QS_SLAB * 64;
        const uint64_t group0 = static_cast<uint64_t>(rt * TILE + slab) * gpr + ct * 8;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int lr = 4 * i + (lane >> 3), gc = lane & 7;
            float v[16];
            unpack16<NVFP4_BF16>(raw[i][0], raw[i][1], v);
            if constexpr (R_RHT) hadamard16_unscaled(v, sg);
            const uint64_t group = group0 + static_cast<uint32_t>(lr * static_cast<int>(gpr) + gc);
            uint32_t sb;
            const uint2 p = encode16<SR, FAST>(v, R_RHT, inv, seed, static_cast<uint32_t>(group) << 4, group, sb);
            *reinterpret_cast<uint2*>(out + lr * 64 + gc * 8) = p;
            out_sc[lr * 8 + gc] = static_cast<uint8_t>(sb);
        }
        fence_async_shared();
        __syncwarp();
        {
            const int piece_row = slab + (lane >> 1), piece_half = lane & 1;
            const uint32_t piece = *reinterpret_cast<const uint32_t*>(out_sc + (lane >> 1) * 8 + piece_half * 4);
            *reinterpret_cast<uint32_t*>(a.R.scales + (static_cast<int64_t>(rt) * (a.R.kp >> 6) + ct * 2) * 512 + piece_half * 512 +
                                         (piece_row & 31) * 16 + (piece_row >> 5) * 4) = piece;
        }
        if (lane == 0) {
            tma_store_2d(map_row, ct * 64, rt * TILE + slab, out);
            bulk_commit();
        }
    }
    if (lane == 0) bulk_wait_all();
}

template <int SR, bool R_RHT>
__global__ void __launch_bounds__(QR_THREADS, 1)
quant_resident_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_row, const ResidentArgs a) {
    using namespace aop;
    extern __shared__ __align__(128) uint8_t resident_smem_raw[];
    ResidentSmem& S = *reinterpret_cast<ResidentSmem*>(resident_smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_tiles = a.tiles_r * a.tiles_c;
    const int my_tiles = (n_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    if (tid == 0) {
        for (int k = 0; k < my_tiles; ++k) mbar_init(&S.full[k], 1);
        S.abort = 0;
        fence_barrier_init();
        for (int k = 0; k < my_tiles; ++k) {
            const int t = blockIdx.x + k * gridDim.x;
            const int rt = t / a.tiles_c, ct = t - rt * a.tiles_c;
            mbar_expect_tx(&S.full[k], QS_TILE_BYTES);
            tma_load_2d(S.in[k], &map_in, ct * TILE, rt * TILE, &S.full[k]);
        }
    }
    __syncthreads();
    // ---- phase 1: magnitude maximum of this CTA's tiles (|bf16| orders like its 15 magnitude bits) ----
    uint32_t best2 = 0;
    bool landed = true;
    for (int k = 0; k < my_tiles && landed; ++k) {
        landed = __all_sync(0xffffffffu, mbar_wait(&S.full[k], 0, &S.abort));
        if (!landed) break;
        const uint4* p = reinterpret_cast<const uint4*>(S.in[k]) + warp * 128 + lane;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 q = p[32 * j];
            best2 = __vmaxu2(best2, q.x & 0x7fff7fffu); best2 = __vmaxu2(best2, q.y & 0x7fff7fffu);
            best2 = __vmaxu2(best2, q.z & 0x7fff7fffu); best2 = __vmaxu2(best2, q.w & 0x7fff7fffu);
        }
    }
    uint32_t best = max(best2 & 0xffffu, best2 >> 16);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, d));
    if (lane == 0) S.warp_best[warp] = best;
    __syncthreads();
    // ---- grid barrier: the global maximum is complete after it ----
    if (tid == 0) {
        uint32_t b = 0;
        for (int w = 0; w < QR_WARPS; ++w) b = max(b, S.warp_best[w]);
        atomicMax(a.amax_word, b);
        __threadfence();
        atomicAdd(a.arrivals, 1u);
        const long long t0 = clock64();
        int ok = S.abort ? 0 : 1;
        while (ok && *reinterpret_cast<volatile unsigned int*>(a.arrivals) < gridDim.x) {
            __nanosleep(100);
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) ok = 0;
        }
        __threadfence();
        S.amax_bits = *reinterpret_cast<volatile unsigned int*>(a.amax_word);
        S.proceed = ok;
        if (!ok && a.status) *a.status = NVFP4_ERR_TIMEOUT;
    }
    __syncthreads();
    if (S.proceed) {
        const float amax = __uint_as_float(S.amax_bits << 16);
        const float floor_a = fmaxf(amax, 1.e-12f), c = 1.f / (6.f * 448.f);
        const float plain = __fmul_rn(__fmul_rn(1.f, floor_a), c), rotated = __fmul_rn(__fmul_rn(4.f, floor_a), c);
        const float pts = R_RHT ? rotated : plain;
        if (tid == 0 && blockIdx.x == 0) {
            a.out4[0] = amax; a.out4[1] = plain; a.out4[2] = rotated; a.out4[3] = __fdiv_rn(floor_a, 2688.f);
            *a.R.pts = pts;
        }
        float sg[16];
#pragma unroll
        for (int l = 0; l < 16; ++l) sg[l] = a.signs ? __ldg(a.signs + l) : 1.f;
        const ScaleMath sm = scale_math(pts);
        if (sm.fast) resident_encode<SR, R_RHT, true>(S, &map_row, a, sg, sm.inv, my_tiles, warp, lane);
        else resident_encode<SR, R_RHT, false>(S, &map_row, a, sg, sm.inv, my_tiles, warp, lane);
    }
    // the last CTA to leave zeroes both words for the next launch
    __syncthreads();
    if (tid == 0 && atomicAdd(a.arrivals, 1u) == 2u * gridDim.x - 1u) { *a.amax_word = 0u; __threadfence(); *a.arrivals = 0u; }
}

template <int SR, bool R_RHT>
static cudaError_t launch_resident_one(const CUtensorMap& mi, const CUtensorMap& mr, const ResidentArgs& a, int grid, cudaStream_t st) {
    const size_t smem = sizeof(ResidentSmem);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(quant_resident_kernel<SR, R_RHT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        configured = true;
    }
    void* args[] = {const_cast<CUtensorMap*>(&mi), const_cast<CUtensorMap*>(&mr), const_cast<ResidentArgs*>(&a)};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(quant_resident_kernel<SR, R_RHT>), dim3(grid), dim3(QR_THREADS),
                                       args, smem, st);
}

static bool resident_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("NVFP4_QUANT_RESIDENT");
        on = !(e && e[0] == '0');
    }
    return on != 0;
}

// amax + row packing of a BF16 tensor that fits shared memory.  NVFP4_ERR_UNSUPPORTED: the caller runs the two launches.
static int try_resident(const void* x, int dtype, int64_t rows, int64_t cols, int64_t rs, int64_t cs, const float* signs,
                        const int32_t* base, int flags, uint32_t seed, uint8_t* packed, uint8_t* scales, float* pts_out,
                        void* scratch, int* status, cudaStream_t st) {
    if (!resident_enabled() || !stream_enabled() || dtype != NVFP4_BF16 || cs != 1 || (flags & NVFP4_Q_HI_FIRST)) return NVFP4_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (rs * 2) % 16 != 0 || rs < cols) return NVFP4_ERR_UNSUPPORTED;
    if (((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(scales) | reinterpret_cast<uintptr_t>(scratch)) & 15) != 0)
        return NVFP4_ERR_UNSUPPORTED;
    static int sms = 0, coop = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const int64_t rp = round128(rows), cp = round128(cols), tiles = rp / 128 * (cp / 128);
    if (!coop || tiles > static_cast<int64_t>(QR_MAX_TILES) * sms) return NVFP4_ERR_UNSUPPORTED;
    CUtensorMap mi, mr;
    if (!aop::make_map_2d(&mi, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, static_cast<uint64_t>(cols), static_cast<uint64_t>(rows),
                          static_cast<uint64_t>(rs) * 2, TILE, TILE))
        return NVFP4_ERR_UNSUPPORTED;
    if (!aop::make_map_2d(&mr, CU_TENSOR_MAP_DATA_TYPE_UINT8, packed, static_cast<uint64_t>(cp / 2), static_cast<uint64_t>(rp),
                          static_cast<uint64_t>(cp / 2), 64, QS_SLAB))
        return NVFP4_ERR_UNSUPPORTED;
    char* sc = static_cast<char*>(scratch);
    ResidentArgs a{signs, base, reinterpret_cast<unsigned int*>(sc + SCRATCH_RESIDENT_OFFSET),
                   reinterpret_cast<unsigned int*>(sc + SCRATCH_RESIDENT_OFFSET + 4),
                   reinterpret_cast<float*>(sc + SCRATCH_AMAX_OUT_OFFSET), status,
                   Orient{packed, scales, pts_out, cp, seed, flags}, static_cast<int>(rp / 128), static_cast<int>(cp / 128)};
    const int grid = static_cast<int>(std::min<int64_t>(tiles, sms));
    const bool rht = flags & NVFP4_Q_RHT;
    const int sr = sr_of_flags(flags);
    cudaError_t e;
    if (sr == SR_NONE) e = rht ? launch_resident_one<SR_NONE, true>(mi, mr, a, grid, st) : launch_resident_one<SR_NONE, false>(mi, mr, a, grid, st);
    else if (sr == SR_HASH) e = rht ? launch_resident_one<SR_HASH, true>(mi, mr, a, grid, st) : launch_resident_one<SR_HASH, false>(mi, mr, a, grid, st);
    else e = rht ? launch_resident_one<SR_PHILOX, true>(mi, mr, a, grid, st) : launch_resident_one<SR_PHILOX, false>(mi, mr, a, grid, st);
    if (e != cudaSuccess) {
        set_error("nvfp4_quantize: cooperative launch of the resident quantiser failed: %s", cudaGetErrorString(e));
        return NVFP4_ERR_LAUNCH;
    }
    return launch_status("nvfp4_quantize");
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
    for (int b = 0; b < 8; ++b) {
        // both codes of a byte in one conversion (e2m1 values are exact in FP16); .x is the low nibble
        const __half2_raw pair = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>((w[b >> 2] >> (8 * (b & 3))) & 0xffu), __NV_E2M1);
        const float lo = __half2float(__ushort_as_half(pair.x)), hi = __half2float(__ushort_as_half(pair.y));
        v[2 * b] = __fmul_rn(__fmul_rn(hi_first ? hi : lo, s), t);
        v[2 * b + 1] = __fmul_rn(__fmul_rn(hi_first ? lo : hi, s), t);
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

static int quantize_tile_impl(const void* x, int dtype, int64_t rows, int64_t cols, int64_t rs, int64_t cs, const float* signs,
                              const int32_t* seed_base, const float* unit, const float* amax, uint8_t* row_packed,
                              uint8_t* row_scales, float* row_pts, int row_flags, uint32_t row_seed, uint8_t* col_packed,
                              uint8_t* col_scales, float* col_pts, int col_flags, uint32_t col_seed, int* status,
                              nvfp4_stream_t stream) {
    NVFP4_REQUIRE(x, NVFP4_ERR_ARG, "nvfp4_quantize_tile: null source");
    NVFP4_REQUIRE(signs || !((row_flags | col_flags) & NVFP4_Q_RHT), NVFP4_ERR_ARG, "nvfp4_quantize_tile: the Hadamard transform needs the sign vector");
    NVFP4_REQUIRE(rows > 0 && cols > 0 && rs >= 0 && cs >= 0, NVFP4_ERR_ARG,
                  "nvfp4_quantize_tile: empty tensor or negative stride (rows=%lld cols=%lld)", (long long)rows, (long long)cols);
    NVFP4_REQUIRE(dtype_ok(dtype) || (dtype == NVFP4_E4M3 && unit), NVFP4_ERR_DTYPE, "nvfp4_quantize_tile: unsupported dtype code %d", dtype);
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
    Orient R{row_packed, row_scales, row_pts, cp, row_seed, row_flags};
    Orient C{col_packed, col_scales, col_pts, rp, col_seed, col_flags};
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int rc = try_stream(x, dtype, rows, cols, rs, cs, signs, amax, seed_base, status, R, C, row, col, st);
    if (rc != NVFP4_ERR_UNSUPPORTED) return rc;
    const int esz = dtype == NVFP4_F32 ? 4 : dtype == NVFP4_E4M3 ? 1 : 2;
    int vec_ok = cs == 1 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (rs * esz) % 16 == 0;
    if (dtype == NVFP4_E4M3) {
        NVFP4_REQUIRE(cs == 1 && rs == cols, NVFP4_ERR_ARG, "nvfp4_quantize_fp8_weight: the weight must be contiguous");
        return launch_tile<NVFP4_E4M3>(x, rows, cols, rs, cs, vec_ok, signs, seed_base, unit, amax, R, C, row, col, st);
    }
    if (dtype == NVFP4_F32) return launch_tile<NVFP4_F32>(x, rows, cols, rs, cs, vec_ok, signs, seed_base, unit, amax, R, C, row, col, st);
    if (dtype == NVFP4_BF16) return launch_tile<NVFP4_BF16>(x, rows, cols, rs, cs, vec_ok, signs, seed_base, unit, amax, R, C, row, col, st);
    return launch_tile<NVFP4_F16>(x, rows, cols, rs, cs, vec_ok, signs, seed_base, unit, amax, R, C, row, col, st);
}

extern "C" int nvfp4_quantize_tile(const void* x, int dtype, int64_t rows, int64_t cols, int64_t rs, int64_t cs,
                                   const float* signs, const int32_t* seed_base, uint8_t* row_packed,
                                   uint8_t* row_scales, const float* row_pts, int row_flags, uint32_t row_seed,
                                   uint8_t* col_packed, uint8_t* col_scales, const float* col_pts, int col_flags,
                                   uint32_t col_seed, int* status, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(dtype != NVFP4_E4M3, NVFP4_ERR_DTYPE, "nvfp4_quantize_tile: E4M3 weights go through nvfp4_quantize_fp8_weight");
    return quantize_tile_impl(x, dtype, rows, cols, rs, cs, signs, seed_base, nullptr, nullptr, row_packed, row_scales,
                              const_cast<float*>(row_pts), row_flags, row_seed, col_packed, col_scales, const_cast<float*>(col_pts),
                              col_flags, col_seed, status, stream);
}

extern "C" int nvfp4_quantize_tile_amax(const void* x, int dtype, int64_t rows, int64_t cols, int64_t rs, int64_t cs,
                                        const float* signs, const int32_t* seed_base, const float* amax, uint8_t* row_packed,
                                        uint8_t* row_scales, float* row_pts, int row_flags, uint32_t row_seed,
                                        uint8_t* col_packed, uint8_t* col_scales, float* col_pts, int col_flags,
                                        uint32_t col_seed, int* status, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(dtype != NVFP4_E4M3, NVFP4_ERR_DTYPE, "nvfp4_quantize_tile_amax: E4M3 weights go through nvfp4_quantize_fp8_weight");
    NVFP4_REQUIRE(amax, NVFP4_ERR_ARG, "nvfp4_quantize_tile_amax: null amax");
    return quantize_tile_impl(x, dtype, rows, cols, rs, cs, signs, seed_base, nullptr, amax, row_packed, row_scales, row_pts,
                              row_flags, row_seed, col_packed, col_scales, col_pts, col_flags, col_seed, status, stream);
}

extern "C" int nvfp4_quantize_fp8_weight(const uint8_t* w, const float* unit, int64_t rows, int64_t cols, const float* pts,
                                         uint8_t* row_packed, uint8_t* row_scales, uint8_t* col_packed, uint8_t* col_scales,
                                         nvfp4_stream_t stream) {
    NVFP4_REQUIRE(w && unit && pts, NVFP4_ERR_ARG, "nvfp4_quantize_fp8_weight: null pointer");
    // no sign vector: this path has no Hadamard transform (every pointer a kernel receives must be a device address)
    return quantize_tile_impl(w, NVFP4_E4M3, rows, cols, cols, 1, nullptr, nullptr, unit, nullptr, row_packed, row_scales,
                              const_cast<float*>(pts), 0, 0, col_packed, col_scales, const_cast<float*>(pts), 0, 0, nullptr, stream);
}

static int quantize_op(const void* x, int dtype, int64_t m, int64_t k, int64_t s0, int64_t s1, int64_t mp, int64_t kp, int sr,
                       int rht, uint32_t seed, const float* signs, const float* given_scale, const int32_t* seed_base, int pair,
                       uint8_t* packed, uint8_t* scales, float* pts_out, uint8_t* packed_t, uint8_t* scales_t, void* scratch,
                       int* status, bool one_launch, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(x && packed && scales && signs, NVFP4_ERR_ARG, "nvfp4_quantize: null pointer");
    NVFP4_REQUIRE(m > 0 && k > 0 && s0 >= 0 && s1 >= 0, NVFP4_ERR_ARG, "nvfp4_quantize: empty/broadcast/negative strides unsupported");
    NVFP4_REQUIRE(mp == round128(m) && kp == round128(k), NVFP4_ERR_ARG,
                  "nvfp4_quantize: padded dimensions must be the sizes rounded up to a multiple of 128");
    NVFP4_REQUIRE(sr == 0 || sr == NVFP4_Q_SR_HASH || sr == NVFP4_Q_SR_PHILOX, NVFP4_ERR_ARG, "nvfp4_quantize: bad sr mode %d", sr);
    NVFP4_REQUIRE(given_scale || (pts_out && scratch), NVFP4_ERR_ARG, "nvfp4_quantize: need pts_out and scratch when no scale is given");
    const float* pts = given_scale;
    if (!given_scale && !pair && s1 == 1 && one_launch) {
        // a tensor that fits shared memory: maximum, scale and packing from one read of the source
        const int rc = try_resident(x, dtype, m, k, s0, s1, signs, seed_base, (rht ? NVFP4_Q_RHT : 0) | sr, seed, packed, scales, pts_out,
                                    scratch, status, reinterpret_cast<cudaStream_t>(stream));
        if (rc != NVFP4_ERR_UNSUPPORTED) return rc;
    }
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
        return nvfp4_quantize_tile(x, dtype, m, k, s0, s1, signs, seed_base, packed, scales, pts, 0, 0, packed_t, scales_t, pts, 0, 0,
                                   status, stream);
    }
    if (s0 == 1 && s1 != 1) {
        // a transposed view of a row-major k x m matrix: its packing is the column orientation of that matrix
        return nvfp4_quantize_tile(x, dtype, k, m, s1, s0, signs, seed_base, nullptr, nullptr, nullptr, 0, 0, packed, scales, pts,
                                   flags, seed, status, stream);
    }
    return nvfp4_quantize_tile(x, dtype, m, k, s0, s1, signs, seed_base, packed, scales, pts, flags, seed, nullptr, nullptr, nullptr,
                               0, 0, status, stream);
}

extern "C" int nvfp4_quantize(const void* x, int dtype, int64_t m, int64_t k, int64_t s0, int64_t s1, int64_t mp,
                              int64_t kp, int sr, int rht, uint32_t seed, const float* signs, const float* given_scale,
                              const int32_t* seed_base, int pair, uint8_t* packed, uint8_t* scales, float* pts_out,
                              uint8_t* packed_t, uint8_t* scales_t, void* scratch, int* status, nvfp4_stream_t stream) {
    return quantize_op(x, dtype, m, k, s0, s1, mp, kp, sr, rht, seed, signs, given_scale, seed_base, pair, packed, scales, pts_out,
                       packed_t, scales_t, scratch, status, true, stream);
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
    return quantize_op(x, dtype, m, k, s0, s1, mp, kp, sr, rht, seed, signs, nullptr, seed_base, 0, packed, scales, pts_out,
                       nullptr, nullptr, scratch, nullptr, false, stream);
}
