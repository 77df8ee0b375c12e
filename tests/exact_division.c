/*
 * Enumeration behind the division-free block-scale arithmetic of the quantiser (csrc/quant_core.cuh: div6_exact,
 * div_e4m3_exact).  With y = rn(1 / b):  q0 = rn(a * y), r = fma(-b, q0, a), q = fma(r, y, q0).
 * Compares q with the IEEE quotient a / b
 *   (1) for b = 6 over non-negative finite floats a, and reports the largest a at which the two differ
 *       (the kernel relies on: none at or above 2^-125);
 *   (2) for every E4M3 value b = 2^e * (1 + m / 8), e in [-6, 8], m in [0, 7], over numerators in [2^-100, 2^100]
 *       (the kernel relies on: no difference at all).
 * Usage: exact_division <stride>   stride 1 walks every bit pattern (about a minute on 8 cores); the test-suite uses a
 * larger odd stride.  Prints two lines: "div6 <mismatches> <largest differing bit pattern>" and "e4m3 <mismatches>".
 * Build: gcc -O2 -fopenmp -ffp-contract=off -mfma tests/exact_division.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static inline float b2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f2b(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

int main(int argc, char** argv) {
    const long long stride = argc > 1 ? atoll(argv[1]) : 1;
    const float c6 = 1.0f / 6.0f;
    long long bad6 = 0;
    uint32_t worst = 0;
#pragma omp parallel
    {
        long long bad = 0;
        uint32_t mine = 0;
#pragma omp for schedule(static)
        for (long long i = 0; i < 0x7f800000LL; i += stride) {
            const float a = b2f((uint32_t)i);
            const float q0 = a * c6;
            const float q = fmaf(fmaf(-6.f, q0, a), c6, q0);
            if (f2b(q) != f2b(a / 6.f)) { ++bad; if ((uint32_t)i > mine) mine = (uint32_t)i; }
        }
#pragma omp critical
        { bad6 += bad; if (mine > worst) worst = mine; }
    }
    printf("div6 %lld %u\n", bad6, worst);
    long long bad8 = 0;
    for (int m = 0; m < 8; ++m) {
        const float mant = 1.f + m / 8.f, rm = 1.0f / mant;
        for (int e = -6; e <= 8; ++e) {
            const float s = ldexpf(mant, e), y = ldexpf(rm, -e);
            long long b = 0;
#pragma omp parallel for reduction(+ : b) schedule(static)
            for (long long i = 0x0d800000LL; i <= 0x71800000LL; i += stride) {   /* 2^-100 .. 2^100 */
                const float a = b2f((uint32_t)i);
                const float q0 = a * y;
                const float q = fmaf(fmaf(-s, q0, a), y, q0);
                if (f2b(q) != f2b(a / s)) ++b;
            }
            bad8 += b;
        }
    }
    printf("e4m3 %lld\n", bad8);
    return 0;
}
