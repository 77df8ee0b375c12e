/*
 * C ABI of libnvfp4_b200.so — hand-written sm_100a CUDA kernels for the NVFP4 training hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream; none allocates and none
 * synchronises.  With one exception none keeps device state of its own, so they are safe under
 * CUDA-graph capture (the quantiser's amax stage uses caller-provided scratch that must start zeroed
 * once and then resets itself).  The exception is nvfp4_quantize_static, whose scratch is an array
 * inside the library image that all its calls on a device share; its comment states the rules that
 * follow from that.  Return value: NVFP4_OK or one of the codes below; nvfp4_last_error() gives the
 * message of the calling thread's last failure.
 *
 * Each declaration names the reference interface it replaces (paths inside the reference project
 * xl03-bit/sm120-nvfp4-training); nvfp4_quantize_static has no counterpart there and says so.
 *
 * `status` arguments: nullable device int that a kernel sets to NVFP4_ERR_TIMEOUT when one of its
 * bounded device-side waits (on an asynchronous copy) gave up; the kernel then returns early
 * instead of hanging.
 */
#ifndef NVFP4_B200_H
#define NVFP4_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* nvfp4_stream_t; /* a cudaStream_t */

enum {
    NVFP4_OK = 0,
    NVFP4_ERR_ARG = 1,         /* null pointer, non-positive size, padded size not a multiple of 128 ... */
    NVFP4_ERR_ALIGN = 2,       /* pointer or stride alignment the kernel needs is not met */
    NVFP4_ERR_DTYPE = 3,       /* unknown element type code */
    NVFP4_ERR_LAUNCH = 4,      /* the CUDA runtime refused the launch (message has the CUDA error) */
    NVFP4_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up (status word written by the kernel) */
    NVFP4_ERR_UNSUPPORTED = 6  /* valid request this build does not implement */
};

/* element type codes */
enum { NVFP4_F32 = 0, NVFP4_BF16 = 1, NVFP4_F16 = 2, NVFP4_E4M3 = 3 };

/* flag bits of nvfp4_gemm's raw_bf16 argument */
enum { NVFP4_GEMM_RAW_BF16 = 1, NVFP4_GEMM_SINGLE_CTA = 2 };

/* per-orientation flags of the quantiser */
enum {
    NVFP4_Q_RHT = 1,        /* sign * H16 / 4 over each 16 contraction elements before scaling */
    NVFP4_Q_SR_HASH = 2,    /* stochastic rounding, the reference's 32-bit integer hash */
    NVFP4_Q_SR_PHILOX = 4,  /* stochastic rounding by the hardware conversion (cvt.rs...e2m1x4) on Philox4x32-10 bits:
                               one block per 16-element group, counter = group index, key = (seed, 0x4e564634) */
    NVFP4_Q_HI_FIRST = 8    /* even element in the high nibble (Comfy checkpoint order) */
};

const char* nvfp4_last_error(void);
int nvfp4_version(void);

/* Number of bytes of zero-initialised scratch nvfp4_amax / nvfp4_quantize need (constant). */
int64_t nvfp4_amax_scratch_bytes(void);

/*
 * max |bf16(x)| of the logical rows x cols view with element strides (row_stride, col_stride),
 * and the tensor scales derived from it:
 *   out[0] = amax
 *   out[1] = (1 * max(amax,1e-12)) * (1/2688)      row / non-RHT scale
 *   out[2] = (4 * max(amax,1e-12)) * (1/2688)      RHT scale
 *   out[3] = max(amax,1e-12) / 2688                true-division variant
 * Replaces reduce_input + finish_reduce (src/nvfp4_training/_backend/csrc/kernels.cu:60-78, launch at
 * :255-275) and _absmax + _scale (src/nvfp4_training/_backend/act_pair.py:9-21).
 */
int nvfp4_amax(const void* x, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int64_t col_stride,
               void* scratch, float* out4, nvfp4_stream_t stream);

/*
 * Tile quantiser: one read of the rows x cols source produces up to two NVFP4 packings.
 *   "row" packing  = packing of x      : row_packed[rows_p][cols_p/2], row_scales swizzled, groups along cols
 *   "col" packing  = packing of x^T    : col_packed[cols_p][rows_p/2], col_scales swizzled, groups along rows
 * rows_p / cols_p are rows / cols rounded up to 128; the padding is written as zeros.  Pass a null
 * packed pointer to skip an orientation.  *_pts point at the FP32 tensor scale on the device,
 * *_flags are NVFP4_Q_* bits, *_seed the SR seed; seed_base (nullable, device int32[1]) is added to
 * both seeds on the device so that CUDA-graph replays draw fresh SR noise.  signs = 16 device floats.
 * BF16 / FP16 sources with unit column stride and 16-byte aligned rows run on the persistent streaming kernel (TMA tile
 * loads, TMA / bulk stores); every other source on a kernel with per-thread loads.  Same results.
 * Replaces quant_rows / quant_transpose / quant_weight_pair (csrc/kernels.cu:123-185; device-seed
 * variant csrc_graph/kernels.cu:126-127), _dual (act_pair.py:50-71), _pair (pair.py:25-36) and _single
 * (remat.py:7-19).
 */
int nvfp4_quantize_tile(const void* x, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int64_t col_stride,
                        const float* signs, const int32_t* seed_base,
                        uint8_t* row_packed, uint8_t* row_scales, const float* row_pts, int row_flags, uint32_t row_seed,
                        uint8_t* col_packed, uint8_t* col_scales, const float* col_pts, int col_flags, uint32_t col_seed,
                        int* status, nvfp4_stream_t stream);

/*
 * nvfp4_quantize_tile for a source whose producer left its amax on the device (a kernel of this library that ends in an
 * atomic maximum, see the workload helpers below): the tensor scales are computed inside the quantiser as
 * (factor * max(amax[0], 1e-12)) * (1 / 2688), factor 4 for an orientation under the Hadamard transform, 1 otherwise, and
 * written to row_pts / col_pts; no separate pass over the source.  Same results as nvfp4_amax + nvfp4_quantize_tile, which
 * replace _absmax + _scale + _dual (src/nvfp4_training/_backend/act_pair.py:9-21,50-71).
 */
int nvfp4_quantize_tile_amax(const void* x, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int64_t col_stride,
                             const float* signs, const int32_t* seed_base, const float* amax,
                             uint8_t* row_packed, uint8_t* row_scales, float* row_pts, int row_flags, uint32_t row_seed,
                             uint8_t* col_packed, uint8_t* col_scales, float* col_pts, int col_flags, uint32_t col_seed,
                             int* status, nvfp4_stream_t stream);

/*
 * Both NVFP4 orientations (either may be null) of an FP8 master weight without a dense copy: w [rows][cols] contiguous
 * E4M3 codes, element i worth e4m3(w[i]) * unit[i / 512] rounded to BF16; round to nearest, no Hadamard transform, one
 * tensor scale `pts` for both packings.  Replaces master8._scaled_pair / encode and _decode
 * (src/nvfp4_training/_backend/master8.py:14-23,36-56).
 */
int nvfp4_quantize_fp8_weight(const uint8_t* w, const float* unit, int64_t rows, int64_t cols, const float* pts,
                              uint8_t* row_packed, uint8_t* row_scales, uint8_t* col_packed, uint8_t* col_scales,
                              nvfp4_stream_t stream);

/*
 * The reference's native operator `quantize` (src/nvfp4_training/_backend/csrc/bindings.cpp:9-12 over
 * quantize_cuda, csrc/kernels.cu:237-298): quantise the strided m x k view x into packed[mp][kp/2],
 * scales and pts.  given_scale != null reuses a tensor scale (then pts_out may be null); pair != 0
 * additionally writes the transposed packing (contiguous FP32/FP16/BF16 weights, RNE, no RHT).
 * sr: 0 RNE, NVFP4_Q_SR_HASH or NVFP4_Q_SR_PHILOX.  scratch: nvfp4_amax_scratch_bytes() bytes.
 * Without a given scale the call is two launches (amax, then the quantiser), except for a BF16 source with unit column
 * stride and 16-byte aligned rows of at most 7 x 128 x 128 elements per SM (4096 x 4096 on 148 SMs): that one is loaded
 * into shared memory once and amax, scale and packing come from ONE cooperative launch (same bytes; `status` reports a
 * grid-barrier wait that ran out; the environment variable NVFP4_QUANT_RESIDENT=0 keeps the two launches).
 */
int nvfp4_quantize(const void* x, int dtype, int64_t m, int64_t k, int64_t s0, int64_t s1, int64_t mp, int64_t kp,
                   int sr, int rht, uint32_t seed, const float* signs, const float* given_scale,
                   const int32_t* seed_base, int pair, uint8_t* packed, uint8_t* scales, float* pts_out,
                   uint8_t* packed_t, uint8_t* scales_t, void* scratch, int* status, nvfp4_stream_t stream);

/*
 * nvfp4_quantize for callers that cannot allocate device memory.  No counterpart in the reference project.
 * Some hosts of this library own no allocator they may call at this point: a plug-in running inside another
 * framework's execution callback, a replayed step whose memory plan is frozen, a process whose device memory was handed
 * out up front.  nvfp4_quantize asks such callers for a scratch block they cannot provide; this variant keeps the block
 * (the amax partial maxima, the arrival ticket and the four scale results: 4160 bytes) in a __device__ array inside
 * the library image instead, so every GPU that loads the library holds those 4160 bytes until the process exits.
 * Same arguments and results as nvfp4_quantize without given_scale / pair / scratch; the tensor scale is always
 * computed and written to pts_out.  Tensors above nvfp4_quantize_static_max_elements() (2^31) elements are refused with
 * NVFP4_ERR_ARG.  The call performs no cudaMalloc / cudaFree and uses no allocating library routine.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call outside any stream capture.  All calls on a device share the one array: calls that
 * may overlap on the GPU (different streams, no ordering) race on it and must be serialised by the caller.  The address
 * look-up itself is not synchronised: make the first call per device from one host thread.
 */
int64_t nvfp4_quantize_static_max_elements(void);
int nvfp4_quantize_static(const void* x, int dtype, int64_t m, int64_t k, int64_t s0, int64_t s1, int64_t mp, int64_t kp,
                          int sr, int rht, uint32_t seed, const float* signs, const int32_t* seed_base, uint8_t* packed,
                          uint8_t* scales, float* pts_out, nvfp4_stream_t stream);

/*
 * NVFP4 -> FP32 or BF16: out[r][c] = (level * block_scale) * pts for r < rows, c < cols.
 * Replaces dequant (src/precision_lora/_packed_cuda.py:56-63) and the TorchAO NVFP4Tensor.dequantize used
 * by the reference's verifier (src/nvfp4_training/_verification/nvfp4_cuda.py:184-200).
 */
int nvfp4_dequantize(const uint8_t* packed, const uint8_t* scales, const float* pts, int64_t kp, int64_t rows,
                     int64_t cols, int hi_first, int out_dtype, void* out, int64_t out_stride, nvfp4_stream_t stream);

/*
 * Block-scaled NVFP4 GEMM with fused epilogue:  out[rows x cols] = crop((A o SFA) (B o SFB)^T) * alpha (+ bias).
 *   a [M][K/2], b [N][K/2]: e2m1 payloads (low nibble = even element), K-major; sfa, sfb: swizzled ue4m3 block
 *   scales as the quantiser writes them; M, N, K multiples of 128; FP32 accumulation (tcgen05, TMEM).
 *   pts_a, pts_b: device FP32 tensor scales, alpha = pts_a * pts_b; both null = store the raw accumulator.
 *   raw_bf16 is a flag word.  Bit 0 set reproduces the reference's BF16 chain: bf16(acc), alpha -> bf16,
 *   bf16(raw * alpha), bf16(y + bf16(bias)); bit 0 clear is the FP32 chain acc * alpha (+ bias).
 *   NVFP4_GEMM_SINGLE_CTA (bit 1) keeps every tile on one SM; by default shapes with M and N multiples of 256 run on
 *   pairs of SMs (thread-block clusters of two, 256-row MMAs), which gives the same results.
 *   out: FP32 or BF16, row stride ldo elements.  status: nullable device int, set to NVFP4_ERR_TIMEOUT if a
 *   bounded device-side wait expired (the kernel then returns early instead of hanging).
 * Replaces torch._scaled_mm on float4_e2m1fn_x2 operands (src/nvfp4_training/_backend/nvfp4_fast_v2.py:208-215,
 * scale6.py:35-37, nvfp4_v5.py:122-125, linear6.py:141-144; src/precision_lora/_packed_cuda.py:244-249) together
 * with the separate `rescale` operator (csrc/bindings.cpp:9-12 over rescale_cuda, csrc/kernels.cu:210-234,300-328;
 * scale6.py:7-30).
 */
int nvfp4_gemm(const uint8_t* a, const uint8_t* sfa, const float* pts_a, const uint8_t* b, const uint8_t* sfb,
               const float* pts_b, int64_t M, int64_t N, int64_t K, const void* bias, int bias_dtype, void* out,
               int out_dtype, int64_t ldo, int64_t rows, int64_t cols, int raw_bf16, int* status, nvfp4_stream_t stream);

/*
 * Compressed AdamW step, one kernel per parameter tensor (n elements, flat):
 *   decode master + moments -> m = b1 m + (1-b1) g, v = b2 v + (1-b2) g g,
 *   p = p * decay - (lr c1) m / (sqrt(v) c2 + eps) -> re-encode -> amax of bf16(p) -> next tensor scale.
 * master: 32 FP32 | 24 BF16 head + int8 `tail` | 17 FP16, stochastically rounded | 16 BF16, stochastically rounded |
 *         8 E4M3 times the power-of-two `unit` of each 512 weights (units grow when an update would overflow).
 * moments: mbits 8 = int8 m with FP32 scale per state block; mbits 4 = nibble code (sqrt-coded if nonlinear_m) with
 *          scales per 64; vbits 16 = FP16 v / scale, 8 = uint8 code of sqrt(v), 4 = nibble code of sqrt(v) with scales
 *          per 64 (mbits = vbits = 4: one byte per element in `m`, m low nibble, and `v` is unused).
 * grad_kind: 0 FP32, 1 BF16, 2 raw BF16 GEMM output [*, grad_stride] scaled as bf16(raw * bf16(sa[0] * sb[0])).
 * extra: nullable FP32 gradient added after the decode.  grad_mul: factor applied to the gradient when != 1 (data-
 * parallel averaging).  decay = 1 - lr * weight_decay, c1 = 1 / (1 - b1^t), c2 = 1 / sqrt(1 - b2^t), step = t;
 * ctrl: nullable device float[4] = (c1, c2, -, bits of t) read on the device instead (CUDA-graph replay).
 * key: per-parameter stream of the counter-based rounding bits.  scale_out: nullable device float that receives
 * max(amax, 1e-12) / 2688-by-multiplication, the tensor scale of the next forward; needs `scratch` (the amax scratch).
 * Replaces the Triton kernels adam_kernel.update (src/nvfp4_training/_backend/adam_kernel.py:30-204) and
 * optimizer_v5._partial_max/_finish_scale (optimizer_v5.py:55-64) as launched by AdamW6._update_param
 * (engine6.py:44-104), and master8.round_e4m3 (master8.py:25-34).
 */
int nvfp4_adamw_step(void* p, int master, const void* grad, int grad_kind, int64_t grad_cols, int64_t grad_stride,
                     const float* sa, const float* sb, const float* extra, float grad_mul, void* m, void* v, float* ms,
                     float* vs, int8_t* tail, float* unit, int64_t n, int vbits, int mbits, int nonlinear_m, int state_block,
                     float lr, float decay, float b1, float b2, float c1, float c2, float eps, uint32_t step, uint32_t key,
                     const float* ctrl, float* scale_out, void* scratch, nvfp4_stream_t stream);

/*
 * nvfp4_adamw_step for a weight matrix [rows][cols] that ALSO writes the next forward's two weight packings in the same
 * launch: after the update the kernel's CTAs meet at a grid barrier (cooperative launch, bounded wait, `status` as in
 * nvfp4_gemm) and then quantise the updated master, still resident in L2, against the NEW tensor scale it has just
 * published: packed / scales = the packing of W, packed_t / scales_t that of W^T, round to nearest, byte-identical to
 * nvfp4_quantize(pair = 1) on the updated weight.  Masters FP16 / BF16 (+ tail) / FP32 with the moment formats of the
 * profiles (FP8 masters are refused, as in the reference).  scratch as for nvfp4_adamw_step; scale_out is required.
 * Replaces the FUSE path of adam_kernel.update (src/nvfp4_training/_backend/adam_kernel.py:196-202), whose packings are
 * made with the previous scale and repaired afterwards by prepack._repair (prepack.py:7-37, read at linear6.py:41-55);
 * here the packings are final when the kernel ends.
 */
int nvfp4_adamw_step_prepack(void* p, int master, const void* grad, int grad_kind, int64_t grad_cols, int64_t grad_stride,
                             const float* sa, const float* sb, const float* extra, float grad_mul, void* m, void* v, float* ms,
                             float* vs, int8_t* tail, int64_t rows, int64_t cols, int vbits, int mbits, int nonlinear_m,
                             int state_block, float lr, float decay, float b1, float b2, float c1, float c2, float eps,
                             uint32_t step, uint32_t key, const float* ctrl, float* scale_out, uint8_t* packed, uint8_t* scales,
                             uint8_t* packed_t, uint8_t* scales_t, void* scratch, int* status, nvfp4_stream_t stream);

/*
 * AdamW with FP32 master and FP32 moments for tensors below 4096 elements (norm gains, biases).
 * Replaces optimizer_v5._update with COMPACT = False (src/nvfp4_training/_backend/optimizer_v5.py:9-53).
 */
int nvfp4_adamw_plain(float* p, const float* grad, float* m, float* v, int64_t n, float grad_mul, float lr, float decay,
                      float b1, float b2, float c1, float c2, float eps, const float* ctrl, nvfp4_stream_t stream);

/*
 * FP32 weights -> master storage: FP16 (master 17) or BF16 (16, 24) head, plus the signed int8 residual for 24.
 * Replaces adam_kernel.split_init (src/nvfp4_training/_backend/adam_kernel.py:21-28).
 */
int nvfp4_split_init(const float* src, int64_t n, int master, void* hi, int8_t* tail, nvfp4_stream_t stream);

/*
 * Workload helpers: the BF16 element-wise operations that sit between the NVFP4 layers of the benchmarked decoder, each
 * fused with what surrounds it and with the tensor amax of its result.  `amax` arguments are nullable device floats that
 * must hold 0 (or an earlier maximum) on entry and receive max |result| by an atomic maximum, so that the quantiser of
 * the next NVFP4 layer needs no pass of its own over the tensor (nvfp4_quantize_tile_amax).  The reference keeps a rotary
 * kernel for one of its model integrations (src/precision_lora/_packed_cuda.py:104-114) and otherwise leaves these
 * operations to PyTorch (src/nvfp4_training/_workloads/lm.py).
 *
 * nvfp4_rope: rotary position embedding on [tokens][heads][dim] rows with input / output row pitches in elements (split-
 * half convention, tables cos / sin [seq][dim / 2]); mode 0 rotates, 1 applies the inverse rotation (the backward pass),
 * 2 copies (the un-rotated part of a fused q / k / v gradient).
 * nvfp4_swiglu: out = silu(gate) * up (dout == NULL), or its backward (dgate -> out_or_dgate, dup); every operand is
 * [rows][cols] with its own row pitch, so the halves of a fused gate / up projection are used in place.
 * nvfp4_add_rmsnorm: sum = x + delta (skipped when delta == NULL), h = sum * rsqrt(mean(sum^2) + eps) * bf16(gamma),
 * rstd kept for the backward pass.
 * nvfp4_rmsnorm_bwd: dx = d(h -> sum) + dres (dres nullable: the gradient arriving on the residual path) and dgamma;
 * `partial` is FP32 scratch of nvfp4_rmsnorm_bwd_partials(rows, cols) x cols elements, reduced in a fixed order.
 */
int nvfp4_rope(const void* x, void* out, const void* cos_t, const void* sin_t, int64_t tokens, int seq, int heads, int dim,
               int64_t pitch, int64_t out_pitch, int mode, float* amax, nvfp4_stream_t stream);
/* The backward pass of nvfp4_rope over a fused q / k / v projection in one launch: dqkv [tokens][3 * heads * dim] receives the
 * inverse rotation of dq and dk and a copy of dv (each [tokens][heads][dim] with its own row pitch); amax as above. */
int nvfp4_rope_qkv_bwd(const void* dq, int64_t dq_pitch, const void* dk, int64_t dk_pitch, const void* dv, int64_t dv_pitch,
                       void* dqkv, const void* cos_t, const void* sin_t, int64_t tokens, int seq, int heads, int dim,
                       float* amax, nvfp4_stream_t stream);
int nvfp4_swiglu(const void* gate, int64_t gate_pitch, const void* up, int64_t up_pitch, const void* dout, int64_t dout_pitch,
                 void* out_or_dgate, int64_t out_pitch, void* dup, int64_t dup_pitch, int64_t rows, int64_t cols, float* amax,
                 nvfp4_stream_t stream);
int nvfp4_add_rmsnorm(const void* x, const void* delta, const float* gamma, float eps, int64_t rows, int64_t cols, void* sum_out,
                      void* h_out, float* rstd_out, float* amax_out, nvfp4_stream_t stream);
int64_t nvfp4_rmsnorm_bwd_partials(int64_t rows, int64_t cols);
int nvfp4_rmsnorm_bwd(const void* dh, const void* sum, const float* rstd, const float* gamma, const void* dres, int64_t rows,
                      int64_t cols, void* dx, float* partial, float* dgamma, float* amax_out, nvfp4_stream_t stream);

/*
 * Mean token cross-entropy over BF16 logits [rows][cols] (row pitch in elements; cols a multiple of 8, at most 32768),
 * int64 targets; FP32 math.  fwd: lse[rows] (kept for the backward pass), row_loss[rows] (scratch), loss = mean over rows,
 * added in a fixed order.  bwd: dlogits = (softmax - onehot) * grad_out[0] / rows, rounded once to BF16, with max |dlogits|
 * left in `amax` (nullable) for the quantiser of the output projection's backward.  The reference's benchmark model takes
 * torch.nn.functional.cross_entropy on an FP32 copy of the logits (src/nvfp4_training/_workloads/lm.py); its optional
 * Triton loss (token_loss.py) is a different fusion and not what this replaces.
 */
int nvfp4_cross_entropy_fwd(const void* logits, int64_t pitch, const int64_t* targets, int64_t rows, int64_t cols, float* lse,
                            float* row_loss, float* loss, nvfp4_stream_t stream);
int nvfp4_cross_entropy_bwd(const void* logits, int64_t pitch, const int64_t* targets, const float* lse, const float* grad_out,
                            int64_t rows, int64_t cols, void* dlogits, int64_t out_pitch, float* amax, nvfp4_stream_t stream);

/*
 * ---- frozen NVFP4 checkpoints in "Comfy" order as LoRA bases ------------------------------------------------------
 * Payload bytes hold the even element in the HIGH nibble; block scales are E4M3 in the same 128 x 4 swizzle as above;
 * one FP32 tensor scale.  These five entry points replace the run-time-compiled kernels the reference launches through
 * the CUDA driver API (src/precision_lora/_packed_cuda.py:215-219, `launch(name, blocks, threads, *args)`).
 *
 * nvfp4_comfy_quantize: x [rows][cols] BF16 contiguous, cols % 128 == 0.  With signs128 != NULL every aligned run of
 * 128 columns is first rotated by sign * H128 / sqrt(128).  tensor_scale[0] = max(amax / 2688, 1e-30); block scales are
 * the software E4M3 RNE of max16 / (6 * tensor_scale); elements are rounded by the hardware RNE conversion, or with
 * sr != 0 stochastically from mix32(element index ^ (seed + counter[0])) (counter nullable, device int32).  Writes
 * packed [ceil16(rows)][cols / 2], scales for ceil128(rows) rows (rows past `rows` as zeros) and tensor_scale.
 * amax_scratch: one device float, overwritten.  Replaces kernels rotate, amax_bf16 and quant (_packed_cuda.py:64-103)
 * and their launcher quantize() (:228-243).
 */
int nvfp4_comfy_quantize(const void* x, int64_t rows, int64_t cols, const float* signs128, int sr, uint32_t seed,
                         const int32_t* counter, uint8_t* packed, uint8_t* scales, float* tensor_scale, float* amax_scratch,
                         nvfp4_stream_t stream);

/* packed [n][k / 2] -> BF16 [n][k]: scale = bf16(g * e4m3(s)), value = bf16(e2m1 * scale).  k % 16 == 0.
 * Replaces kernel dequant (_packed_cuda.py:56-63, launcher :221-225). */
int nvfp4_comfy_dequantize(const uint8_t* packed, const uint8_t* scales, const float* tensor_scale, void* out, int64_t n,
                           int64_t k, nvfp4_stream_t stream);

/*
 * The input-gradient operand of a packed weight W [n][k] without a dense copy: decode, multiply by signs128 along n,
 * rotate each aligned run of 128 output features by H128 / sqrt(128), requantise (RNE) as [k][n].  n, k % 128 == 0.
 * nvfp4_comfy_backward_scale computes that tensor's scale max(amax / 2688, 1e-30) (amax_scratch: one device float,
 * overwritten); nvfp4_comfy_transpose_requant writes packed_t [k][n / 2] and scales_t against a given scale.
 * Replace kernel transpose_rht_quant in its two modes and finish_scale (_packed_cuda.py:81-83,117-163; launchers
 * transpose_rht_quant :266-273 and backward_scale :276-287).
 */
int nvfp4_comfy_backward_scale(const uint8_t* packed, const uint8_t* scales, const float* tensor_scale, const float* signs128,
                               int64_t n, int64_t k, float* amax_scratch, float* backward_scale, nvfp4_stream_t stream);
int nvfp4_comfy_transpose_requant(const uint8_t* packed, const uint8_t* scales, const float* tensor_scale,
                                  const float* signs128, const float* backward_scale, uint8_t* packed_t, uint8_t* scales_t,
                                  int64_t n, int64_t k, nvfp4_stream_t stream);
/* scale[0] = max(amax[0] / 2688, 1e-30) with an IEEE division on the device (_packed_cuda.py:81-83). */
int nvfp4_comfy_finish_scale(const float* amax, float* scale, nvfp4_stream_t stream);

/*
 * Rotary embedding by per-row 2 x 2 matrices: x, out [rows][heads][dim] BF16, rotation [rows][pairs][2][2] BF16; feature
 * pairs (p, p + pairs) are multiplied by the matrix (its transpose when backward != 0), features from 2 * pairs on are
 * copied.  Replaces kernel rope (_packed_cuda.py:104-114, launcher :251-257).
 */
int nvfp4_comfy_rope(const void* x, const void* rotation, void* out, int64_t rows, int heads, int dim, int pairs, int backward,
                     nvfp4_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
