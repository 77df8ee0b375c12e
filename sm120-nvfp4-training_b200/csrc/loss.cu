// Token cross-entropy over BF16 logits for the decoder workload: one pass for the loss (row maximum, log-sum-exp, the
// target's logit), one pass for the gradient (softmax minus one-hot, scaled, rounded once to BF16, with the tensor amax
// for the quantiser of the output projection's backward).  A CTA owns a row; the row is held in registers between the
// maximum and the sum, so each pass reads the logits once.  FP32 math with expf / logf, as torch's log_softmax on the FP32
// copy of the logits that this replaces.
#include "bf16x8.cuh"

#include <algorithm>

namespace nvfp4 {

constexpr int CE_THREADS = 256;
constexpr int CE_CHUNKS = 16;                        // 16-byte chunks per thread: rows of up to 256 * 16 * 8 = 32768 logits
constexpr float CE_LOWEST = -3.0e38f;

__device__ __forceinline__ float block_reduce(float v, bool take_max, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = take_max ? warp_max(v) : warp_sum(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = scratch[0];
#pragma unroll
    for (int w = 1; w < CE_THREADS / 32; ++w) total = take_max ? fmaxf(total, scratch[w]) : total + scratch[w];   // fixed order
    __syncthreads();
    return total;
}

// The row of one CTA, chunk c of thread t being columns (c * 256 + t) * 8 ..; absent chunks are filled with CE_LOWEST.
__device__ __forceinline__ void load_row(const uint16_t* row, int chunks, uint4 (&raw)[CE_CHUNKS]) {
    const uint4 lowest = make_uint4(0xff7fff7fu, 0xff7fff7fu, 0xff7fff7fu, 0xff7fff7fu);   // eight times -3.39e38
#pragma unroll
    for (int c = 0; c < CE_CHUNKS; ++c) {
        const int at = c * CE_THREADS + threadIdx.x;
        raw[c] = at < chunks ? reinterpret_cast<const uint4*>(row)[at] : lowest;
    }
}

__device__ __forceinline__ float row_lse(const uint4 (&raw)[CE_CHUNKS], float* scratch) {
    float best = CE_LOWEST;
#pragma unroll
    for (int c = 0; c < CE_CHUNKS; ++c) {
        float v[8];
        unpack8(raw[c], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) best = fmaxf(best, v[j]);
    }
    best = block_reduce(best, true, scratch);
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < CE_CHUNKS; ++c) {
        float v[8];
        unpack8(raw[c], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += expf(v[j] - best);      // the fill value contributes exp(-inf-like) = 0
    }
    sum = block_reduce(sum, false, scratch);
    return best + logf(sum);
}

__global__ void __launch_bounds__(CE_THREADS, 2) ce_forward_kernel(const uint16_t* __restrict__ logits, int64_t pitch,
                                                                const int64_t* __restrict__ targets, int cols,
                                                                float* __restrict__ lse_out, float* __restrict__ row_loss) {
    __shared__ float scratch[CE_THREADS / 32];
    const int64_t r = blockIdx.x;
    const uint16_t* row = logits + r * pitch;
    uint4 raw[CE_CHUNKS];
    load_row(row, cols / 8, raw);
    const float lse = row_lse(raw, scratch);
    if (threadIdx.x == 0) {
        const int64_t t = targets[r];
        const bool valid = t >= 0 && t < cols;
        lse_out[r] = lse;
        row_loss[r] = valid ? lse - bf16_value(row[t]) : 0.f;
    }
}

// mean of the row losses in a fixed order (one CTA)
__global__ void __launch_bounds__(1024) ce_mean_kernel(const float* __restrict__ row_loss, int64_t rows, float* __restrict__ out) {
    __shared__ float part[1024];
    float t = 0.f;
    for (int64_t i = threadIdx.x; i < rows; i += 1024) t += row_loss[i];
    part[threadIdx.x] = t;
    __syncthreads();
    for (int step = 512; step > 0; step >>= 1) {
        if (threadIdx.x < step) part[threadIdx.x] += part[threadIdx.x + step];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[0] = part[0] / static_cast<float>(rows);
}

__global__ void __launch_bounds__(CE_THREADS, 2) ce_backward_kernel(const uint16_t* __restrict__ logits, int64_t pitch,
                                                                 const int64_t* __restrict__ targets, const float* __restrict__ lse,
                                                                 const float* __restrict__ grad_out, int64_t rows, int cols,
                                                                 uint16_t* __restrict__ dlogits, int64_t out_pitch,
                                                                 float* __restrict__ amax) {
    const int64_t r = blockIdx.x;
    const int chunks = cols / 8;
    uint4 raw[CE_CHUNKS];
    load_row(logits + r * pitch, chunks, raw);
    const float shift = lse[r];
    const float scale = grad_out[0] / static_cast<float>(rows);
    const int64_t t = targets[r];
    float best = 0.f;
#pragma unroll
    for (int c = 0; c < CE_CHUNKS; ++c) {
        const int at = c * CE_THREADS + threadIdx.x;
        if (at >= chunks) break;
        float v[8], g[8];
        unpack8(raw[c], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float p = expf(v[j] - shift);
            g[j] = (at * 8 + j == t ? p - 1.f : p) * scale;
        }
        const uint4 packed = pack8(g);
        reinterpret_cast<uint4*>(dlogits + r * out_pitch)[at] = packed;
        best = fmaxf(best, abs_max8(packed));
    }
    block_atomic_amax(amax, best);
}

}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_cross_entropy_fwd(const void* logits, int64_t pitch, const int64_t* targets, int64_t rows, int64_t cols,
                                       float* lse, float* row_loss, float* loss, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(logits && targets && lse && row_loss && loss, NVFP4_ERR_ARG, "nvfp4_cross_entropy_fwd: null pointer");
    NVFP4_REQUIRE(rows > 0 && cols > 0 && cols % 8 == 0 && cols <= CE_THREADS * CE_CHUNKS * 8 && pitch >= cols && pitch % 8 == 0,
                  NVFP4_ERR_ARG, "nvfp4_cross_entropy_fwd: columns must be a multiple of 8, at most %d, pitch a multiple of 8",
                  CE_THREADS * CE_CHUNKS * 8);
    NVFP4_REQUIRE((reinterpret_cast<uintptr_t>(logits) & 15) == 0, NVFP4_ERR_ALIGN, "nvfp4_cross_entropy_fwd: logits must be 16-byte aligned");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    ce_forward_kernel<<<static_cast<unsigned>(rows), CE_THREADS, 0, st>>>(static_cast<const uint16_t*>(logits), pitch, targets,
                                                                          static_cast<int>(cols), lse, row_loss);
    ce_mean_kernel<<<1, 1024, 0, st>>>(row_loss, rows, loss);
    return launch_status("nvfp4_cross_entropy_fwd");
}

extern "C" int nvfp4_cross_entropy_bwd(const void* logits, int64_t pitch, const int64_t* targets, const float* lse,
                                       const float* grad_out, int64_t rows, int64_t cols, void* dlogits, int64_t out_pitch,
                                       float* amax, nvfp4_stream_t stream) {
    NVFP4_REQUIRE(logits && targets && lse && grad_out && dlogits, NVFP4_ERR_ARG, "nvfp4_cross_entropy_bwd: null pointer");
    NVFP4_REQUIRE(rows > 0 && cols > 0 && cols % 8 == 0 && cols <= CE_THREADS * CE_CHUNKS * 8 && pitch >= cols && pitch % 8 == 0 &&
                      out_pitch >= cols && out_pitch % 8 == 0,
                  NVFP4_ERR_ARG, "nvfp4_cross_entropy_bwd: columns must be a multiple of 8, at most %d, pitches multiples of 8",
                  CE_THREADS * CE_CHUNKS * 8);
    NVFP4_REQUIRE(((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(dlogits)) & 15) == 0, NVFP4_ERR_ALIGN,
                  "nvfp4_cross_entropy_bwd: tensors must be 16-byte aligned");
    ce_backward_kernel<<<static_cast<unsigned>(rows), CE_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(logits), pitch, targets, lse, grad_out, rows, static_cast<int>(cols),
        static_cast<uint16_t*>(dlogits), out_pitch, amax);
    return launch_status("nvfp4_cross_entropy_bwd");
}
