// Test program (not part of the library): compares SharedDivisor, the FMA division by a block's shared scale used in the
// AdamW kernels, with the IEEE quotient a / b on a GPU.  Prints "mismatches <count> of <cases>".
//   divisors: every `stride`-th float mantissa at three exponents inside the safe range, all-ones and all-zero mantissas
//   numerators per divisor: quotients at and next to the rounding boundaries the kernels care about (k + 1/2 for the int8
//   code, midpoints between neighbouring floats for everything else), plus pseudo-random quotients in [2^-43, 32768].
#include "common.cuh"
#include <cstdio>
#include <cstdlib>

using namespace nvfp4;

__device__ unsigned long long g_bad, g_cases;

__device__ __forceinline__ void check(const SharedDivisor& d, float a, unsigned long long& bad, unsigned long long& cases) {
    const float want = __fdiv_rn(a, d.b);
    if (!(fabsf(want) >= 1.1368683772161603e-13f && fabsf(want) <= 32768.f)) return;   // the stated domain: 2^-43 .. 32768
    ++cases;
    if (__float_as_uint(d(a)) != __float_as_uint(want)) ++bad;
}

__global__ void probe(unsigned stride, unsigned per_divisor) {
    const unsigned long long tid = blockIdx.x * static_cast<unsigned long long>(blockDim.x) + threadIdx.x;
    const unsigned long long mant = tid * stride;
    if (mant >= (1ull << 23)) return;
    unsigned long long bad = 0, cases = 0;
    const int exps[3] = {127 - 50, 127, 127 + 40};
    for (int e = 0; e < 3; ++e) {
        for (int special = 0; special < 3; ++special) {
            const unsigned m = special == 0 ? static_cast<unsigned>(mant) : special == 1 ? 0x7fffffu : 0u;
            if (special && tid) continue;
            const float b = __uint_as_float((static_cast<unsigned>(exps[e]) << 23) | m);
            const SharedDivisor d = shared_divisor(b);
            if (!d.safe) { ++bad; continue; }
            // half-integers k + 1/2, the turning points of the int8 momentum code
            for (int k = 0; k < 127; ++k) {
                const float centre = __fmul_rn(static_cast<float>(k) + 0.5f, b);
                for (int off = -2; off <= 2; ++off) check(d, __uint_as_float(__float_as_uint(centre) + off), bad, cases);
            }
            // midpoints between neighbouring floats of pseudo-random quotients
            unsigned rng = mix32(static_cast<unsigned>(mant) * 2654435761u + e * 977u + special);
            for (unsigned i = 0; i < per_divisor; ++i) {
                rng = mix32(rng + i);
                const unsigned qe = 127 - 43 + rng % 58;                 // exponent of the quotient: 2^-43 .. 2^14
                const float q = __uint_as_float((qe << 23) | (mix32(rng) & 0x7fffffu));
                const double mid = static_cast<double>(q) + 0.5 * static_cast<double>(__uint_as_float((qe << 23)) ) * 1.1920928955078125e-07;
                const float a0 = __double2float_rn(mid * static_cast<double>(b));
                for (int off = -1; off <= 1; ++off) {
                    check(d, __uint_as_float(__float_as_uint(a0) + off), bad, cases);
                    check(d, -__uint_as_float(__float_as_uint(a0) + off), bad, cases);
                }
                check(d, __fmul_rn(q, b), bad, cases);
            }
        }
    }
    atomicAdd(&g_bad, bad);
    atomicAdd(&g_cases, cases);
}

int main(int argc, char** argv) {
    const unsigned stride = argc > 1 ? static_cast<unsigned>(atoi(argv[1])) : 64;
    const unsigned per = argc > 2 ? static_cast<unsigned>(atoi(argv[2])) : 64;
    const unsigned long long zero = 0;
    cudaMemcpyToSymbol(g_bad, &zero, sizeof(zero));
    cudaMemcpyToSymbol(g_cases, &zero, sizeof(zero));
    const unsigned long long threads = ((1ull << 23) + stride - 1) / stride;
    probe<<<static_cast<unsigned>((threads + 127) / 128), 128>>>(stride, per);
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("error %s\n", cudaGetErrorString(cudaGetLastError())); return 1; }
    unsigned long long bad = 0, cases = 0;
    cudaMemcpyFromSymbol(&bad, g_bad, sizeof(bad));
    cudaMemcpyFromSymbol(&cases, g_cases, sizeof(cases));
    printf("mismatches %llu of %llu\n", bad, cases);
    return 0;
}
