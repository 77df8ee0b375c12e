/*
 * CPU restatement of the packed-checkpoint ("Comfy" order) NVFP4 LoRA backend.  TEST INFRASTRUCTURE ONLY: the checker
 * of the CUDA kernels in csrc/comfy.cu; no product code path may call it.
 *
 * Each function follows a numbered place of the reference project (paths relative to its root):
 *   bf / rb (BF16 decode, integer RNE)       src/precision_lora/_packed_cuda.py:14-17
 *   f8 / rf8 (E4M3 decode, software RNE)     src/precision_lora/_packed_cuda.py:18-31
 *   f4 / rf4 (E2M1 decode, RNE / SR encode)  src/precision_lora/_packed_cuda.py:32-47
 *   mix                                      src/precision_lora/_packed_cuda.py:37
 *   swizzle                                  src/precision_lora/_packed_cuda.py:53-55
 *   dequant                                  src/precision_lora/_packed_cuda.py:56-63
 *   rotate (sign * H128 / sqrt 128) + amax   src/precision_lora/_packed_cuda.py:64-80
 *   finish_scale                             src/precision_lora/_packed_cuda.py:81-83
 *   quant                                    src/precision_lora/_packed_cuda.py:84-103 and the launcher :228-243
 *   rope                                     src/precision_lora/_packed_cuda.py:104-114
 *   transpose_rht_quant (both modes)         src/precision_lora/_packed_cuda.py:117-163
 * The reference computes these with one GPU thread per element and warp shuffles; here the same per-element
 * arithmetic is written as plain loops (the butterfly "partner minus self when the index bit is set" becomes an index
 * loop), one IEEE FP32 rounding per operation (-ffp-contract=off mirrors the reference's --fmad=false).
 *
 * Parity status: the scalar functions are pinned bit for bit against the reference's own device functions, compiled
 * as host C++ from the reference source by tests/golden/make_golden_comfy.py (fixture comfy_scalar_reference.npz).
 * The kernels built from them cannot execute without an SM120 GPU and the reference ships no byte vectors for them, so
 * their composition is pinned only through the relations the reference's tests state: finish_scale equals the
 * correctly rounded float64 quotient, transpose-requantise equals quantise(dequantise(W)^T), cache equals recompute.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

uint8_t orc_f32_to_e2m1_rne(float v);   /* nvfp4_oracle.c: the hardware cvt.rn.satfinite.e2m1x2 rounding */

static inline float bits2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f2bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

float orc_comfy_bf(uint16_t x) { return bits2f((uint32_t)x << 16); }
uint16_t orc_comfy_rb(float x) {
    uint32_t u = f2bits(x);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
float orc_comfy_f8(uint8_t x) {
    int e = (x >> 3) & 15, m = x & 7;
    float v = e ? (1.0f + (float)m * 0.125f) * bits2f((uint32_t)(e + 120) << 23) : (float)m * 0.001953125f;
    return (x & 128) ? -v : v;
}
uint8_t orc_comfy_rf8(float v) {
    if (v <= 0.0f) return 0;
    if (v >= 448.0f) return 126;
    int e = (int)((f2bits(v) >> 23) & 255u) - 127;
    if (e < -6) return (uint8_t)lrintf(v * 512.0f);
    int m = (int)lrintf(v * bits2f((uint32_t)(130 - e) << 23)) - 8;
    if (m == 8) { ++e; m = 0; }
    return (uint8_t)(((e + 7) << 3) | m);
}
float orc_comfy_f4(int c) {
    int a = c & 7;
    float v = a < 2 ? (float)a * .5f : bits2f((uint32_t)((a / 2 + 126) << 23) | ((uint32_t)(a & 1) << 22));
    return (c & 8) ? -v : v;
}
uint32_t orc_comfy_mix(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
    return x;
}
/* E2M1 code of v: stochastic between the two adjacent levels, or (sr == 0) software round-to-nearest-even */
uint8_t orc_comfy_rf4(float v, uint32_t rng, int sr) {
    float a = fabsf(v);
    int c = 0;
    if (a >= 6) c = 7;
    else {
        c = (a >= .5f) + (a >= 1.f) + (a >= 1.5f) + (a >= 2.f) + (a >= 3.f) + (a >= 4.f);
        float lo = orc_comfy_f4(c), hi = orc_comfy_f4(c + 1), p = (a - lo) / (hi - lo);
        if (sr ? ((float)(rng >> 8) * 0x1p-24f < p) : (p > .5f || (p == .5f && (c & 1)))) ++c;
    }
    return (uint8_t)(c | (signbit(v) ? 8 : 0));
}
int64_t orc_comfy_swizzle(int64_t r, int64_t b, int64_t k) {
    return (r / 128) * ((k + 63) / 64) * 512 + (b / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + b % 4;
}
float orc_comfy_finish_scale(float amax) { return fmaxf(amax / 2688.0f, 1.0e-30f); }

void orc_comfy_dequantize(const uint8_t* q, const uint8_t* s, float g, uint16_t* y, int64_t n, int64_t k) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r)
        for (int64_t col = 0; col < k; col += 2) {
            uint8_t p = q[(r * k + col) / 2];
            float scale = orc_comfy_bf(orc_comfy_rb(g * orc_comfy_f8(s[orc_comfy_swizzle(r, col / 16, k)])));
            y[r * k + col] = orc_comfy_rb(orc_comfy_f4(p >> 4) * scale);
            y[r * k + col + 1] = orc_comfy_rb(orc_comfy_f4(p & 15) * scale);
        }
}

/* in place: v[j] <- sum over the 128-point sign-Hadamard butterfly, bits 0..6 in order, then * 1/sqrt(128) */
static void hadamard128(float* v) {
    float t[128];
    for (int d = 1; d < 128; d *= 2) {
        for (int j = 0; j < 128; ++j) t[j] = (j & d) ? v[j ^ d] - v[j] : v[j] + v[j ^ d];
        memcpy(v, t, sizeof t);
    }
    for (int j = 0; j < 128; ++j) v[j] *= 0.08838834764831845f;
}

/* y[rows][cols] = rotation of each aligned run of 128 columns of bf16 x times signs; returns amax(|y|) */
float orc_comfy_rotate(const uint16_t* x, const float* signs, float* y, int64_t rows, int64_t cols) {
    float amax = 0.f;
    for (int64_t i = 0; i < rows * cols; i += 128) {
        float v[128];
        for (int j = 0; j < 128; ++j) v[j] = orc_comfy_bf(x[i + j]) * signs[j];
        hadamard128(v);
        for (int j = 0; j < 128; ++j) { y[i + j] = v[j]; amax = fmaxf(amax, fabsf(v[j])); }
    }
    return amax;
}

/* one 16-value group -> scale byte and 16 codes; index = linear element index of the first value */
static uint8_t encode_group(const float* v, float g, int sr, uint32_t seed, int64_t index, uint8_t* codes) {
    float a = 0.f;
    for (int l = 0; l < 16; ++l) a = fmaxf(a, fabsf(v[l]));
    uint8_t sc = orc_comfy_rf8(a / (6.0f * g));
    float tot = orc_comfy_f8(sc) * g;
    for (int l = 0; l < 16; ++l) {
        float normalized = tot == 0 ? 0 : v[l] / tot;
        codes[l] = sr ? orc_comfy_rf4(normalized, orc_comfy_mix((uint32_t)(index + l) ^ seed), 1)
                      : orc_f32_to_e2m1_rne(normalized);
    }
    return sc;
}

/*
 * x [rows][cols] bf16, cols % 128 == 0.  Rows are zero-padded to a multiple of 16 for the payload q [rows16][cols/2];
 * s must hold ceil128(rows) * cols / 16 bytes and is cleared first.  signs == NULL: no rotation.  Returns g.
 */
float orc_comfy_quantize(const uint16_t* x, int64_t rows, int64_t cols, const float* signs, int sr, uint32_t seed,
                         uint8_t* q, uint8_t* s) {
    int64_t rows16 = (rows + 15) / 16 * 16, rows128 = (rows + 127) / 128 * 128;
    float* work = (float*)calloc((size_t)(rows16 * cols), sizeof(float));
    float amax = 0.f;
    if (signs) amax = orc_comfy_rotate(x, signs, work, rows, cols);
    else
        for (int64_t i = 0; i < rows * cols; ++i) { work[i] = orc_comfy_bf(x[i]); amax = fmaxf(amax, fabsf(work[i])); }
    float g = orc_comfy_finish_scale(amax);
    memset(s, 0, (size_t)(rows128 * cols / 16));
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows16; ++r)
        for (int64_t c = 0; c < cols; c += 16) {
            uint8_t codes[16];
            uint8_t sc = encode_group(work + r * cols + c, g, sr, seed, r * cols + c, codes);
            for (int l = 0; l < 16; l += 2) q[(r * cols + c + l) / 2] = (uint8_t)((codes[l] << 4) | codes[l + 1]);
            s[orc_comfy_swizzle(r, c / 16, cols)] = sc;
        }
    free(work);
    return g;
}

/*
 * Packed W [n][k] -> packed rotated W^T [k][n].  backward_global <= 0: only the amax of the rotated transpose is
 * computed (returned); otherwise qt [k][n/2] and st (swizzled, width n) are written and the amax is returned as well.
 */
float orc_comfy_transpose_requant(const uint8_t* q, const uint8_t* s, float g, const float* signs, float backward_global,
                                  uint8_t* qt, uint8_t* st, int64_t n, int64_t k) {
    float amax = 0.f;
    uint16_t* dense = (uint16_t*)malloc((size_t)(n * k) * 2);
    orc_comfy_dequantize(q, s, g, dense, n, k);
    for (int64_t kk = 0; kk < k; ++kk)
        for (int64_t n0 = 0; n0 < n; n0 += 128) {
            float v[128];
            for (int j = 0; j < 128; ++j) v[j] = orc_comfy_bf(dense[(n0 + j) * k + kk]) * signs[j];
            hadamard128(v);
            for (int j = 0; j < 128; ++j) amax = fmaxf(amax, fabsf(v[j]));
            if (backward_global > 0)
                for (int c = 0; c < 128; c += 16) {
                    uint8_t codes[16];
                    uint8_t sc = encode_group(v + c, backward_global, 0, 0, 0, codes);
                    for (int l = 0; l < 16; l += 2)
                        qt[(kk * n + n0 + c + l) / 2] = (uint8_t)((codes[l] << 4) | codes[l + 1]);
                    st[orc_comfy_swizzle(kk, (n0 + c) / 16, n)] = sc;
                }
        }
    free(dense);
    return amax;
}

void orc_comfy_rope(const uint16_t* x, const uint16_t* rot, uint16_t* y, int64_t rows, int heads, int dim, int pairs,
                    int backward) {
    for (int64_t i = 0; i < rows * heads * dim; ++i) {
        int d = (int)(i % dim);
        if (d >= pairs * 2) { y[i] = x[i]; continue; }
        int64_t base = i - d, row = i / ((int64_t)heads * dim);
        int p = d % pairs;
        int64_t offset = (row * pairs + p) * 4;
        float a = orc_comfy_bf(x[base + p]), b = orc_comfy_bf(x[base + p + pairs]);
        float r00 = orc_comfy_bf(rot[offset]), r01 = orc_comfy_bf(rot[offset + 1]);
        float r10 = orc_comfy_bf(rot[offset + 2]), r11 = orc_comfy_bf(rot[offset + 3]);
        float v = backward ? (d < pairs ? a * r00 + b * r10 : a * r01 + b * r11)
                           : (d < pairs ? a * r00 + b * r01 : a * r10 + b * r11);
        y[i] = orc_comfy_rb(v);
    }
}
