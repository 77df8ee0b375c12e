/* Test program: the division-free form of the stochastic round-up test of the AdamW variance code.
 *
 * The kernels store sqrt(v) / scale = z in [0, 255] as an integer code: lo = floor(z), rounded up with probability
 * prob = ((z - lo) * (z + lo)) / (2 lo + 1) (every operation rounded to float), by comparing a 16-bit uniform
 * u = k / 65536 with it:  up = u < prob.  With A = RN((z - lo) * RN(z + lo)) and D = 2 lo + 1 the kernel evaluates
 *     up' = fma(-D, u, A) > D * h(u),   h(u) = half an ulp of u (0 for u = 0),
 * which avoids the division.  This program enumerates z over every float of [0, limit] (every `stride`-th one) for
 * limit = 255 and 15 (the 8-bit and the 4-bit code) and, for each z, the values of k around the turning point of the
 * comparison plus the extremes, and counts the cases where up' differs from up.  Prints "threshold <mismatches> <cases>".
 * Build: gcc -O2 -fopenmp -ffp-contract=off -mfma exact_threshold.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static inline float as_float(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t as_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline int up_reference(float A, float D, uint32_t k) {
    const float u = (float)k * (1.f / 65536.f);
    return u < A / D;
}
static inline int up_new(float A, float D, uint32_t k) {
    const float u = (float)k * (1.f / 65536.f);
    const int32_t hb = (int32_t)(as_bits(u) & 0x7f800000u) - (24 << 23);   /* 2^(e - 24); u = 0 gives a negative pattern */
    const float h = as_float((uint32_t)(hb > 0 ? hb : 0));
    return fmaf(-D, u, A) > D * h;
}

int main(int argc, char** argv) {
    const uint32_t stride = argc > 1 ? (uint32_t)atoi(argv[1]) : 1;
    unsigned long long bad = 0, cases = 0;
    const float limits[2] = {255.f, 15.f};
    for (int which = 0; which < 2; ++which) {
        const uint32_t top = as_bits(limits[which]);
#pragma omp parallel for reduction(+ : bad, cases) schedule(dynamic, 4096)
        for (uint32_t zb = 0; zb <= top; zb += stride) {
            const float z = as_float(zb);
            const float lo = floorf(z);
            const float A = (z - lo) * (z + lo);
            const float D = 2.f * lo + 1.f;
            const float q = A / D;
            const double turn = (double)q * 65536.0;
            const int64_t k0 = (int64_t)floor(turn);
            const int64_t ks[8] = {k0 - 2, k0 - 1, k0, k0 + 1, k0 + 2, 0, 1, 65535};
            for (int i = 0; i < 8; ++i) {
                if (ks[i] < 0 || ks[i] > 65535) continue;
                ++cases;
                bad += up_reference(A, D, (uint32_t)ks[i]) != up_new(A, D, (uint32_t)ks[i]);
            }
        }
    }
    printf("threshold %llu %llu\n", bad, cases);
    return 0;
}
