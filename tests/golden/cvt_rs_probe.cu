// Records what sm_100a's cvt.rs.satfinite.e2m1x4.f32 returns: (1) one non-zero operand at a time against every value of
// every byte of the random word, (2) a million random (x, -x, x/2, 2x, rbits) cases.  Needs a B200:
//     nvcc -gencode arch=compute_100a,code=sm_100a -O2 tests/golden/cvt_rs_probe.cu -o cvt_rs_probe
//     ./cvt_rs_probe <output directory>
// then `python tests/golden/make_golden_cvt_rs.py <output directory>` samples the two dumps into cvt_rs_e2m1x4.npz.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>
#include <cuda_runtime.h>
__global__ void k1(const float* xs, int n, uint16_t* out) {
    // out[((i*4+pos)*4+byte)*256+b]
    long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long total = (long long)n * 4096;
    if (t >= total) return;
    int b = t & 255, byte = (t >> 8) & 3, pos = (t >> 10) & 3; int i = t >> 12;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    v[pos] = xs[i];
    uint32_t r = (uint32_t)b << (8 * byte);
    uint16_t d;
    asm volatile("{ cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5; }" : "=h"(d) : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "r"(r));
    out[t] = d;
}
__global__ void k2(const float* xs, const uint32_t* rs, int n, uint16_t* out) {
    // all four positions share x; arbitrary 32-bit rbits
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    float x = xs[t]; uint32_t r = rs[t];
    uint16_t d;
    asm volatile("{ cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5; }" : "=h"(d) : "f"(x), "f"(-x), "f"(x * 0.5f), "f"(x * 2.f), "r"(r));
    out[t] = d;
}
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); return 1; } } while (0)
int main(int argc, char** argv) {
    std::string dir = argc > 1 ? argv[1] : ".";
    std::vector<float> xs;
    for (int k = 0; k <= 7 * 128; ++k) xs.push_back(k / 128.f);                       // 0..7 step 2^-7
    for (int k = 0; k <= 7 * 128; ++k) xs.push_back(-(k / 128.f));
    for (int k = 0; k < 512; ++k) xs.push_back(1.0f + k / 1024.f + 1.0f / 65536.f);   // fine offsets in [1,1.5)
    for (int k = 0; k < 512; ++k) xs.push_back(k / 1024.f + 1.0f / 1048576.f);        // [0,.5)
    for (int k = 0; k < 512; ++k) xs.push_back(4.f + k / 256.f + 1.0f / 16384.f);     // [4,6)
    for (int k = 0; k < 512; ++k) xs.push_back(2.f + k / 256.f + 1.0f / 32768.f);     // [2,4)
    for (int k = 0; k < 64; ++k) xs.push_back(ldexpf(1.f, -k));                       // tiny
    int n = (int)xs.size();
    float* dx; uint16_t* dout;
    CK(cudaMalloc(&dx, n * 4)); CK(cudaMalloc(&dout, (size_t)n * 4096 * 2));
    CK(cudaMemcpy(dx, xs.data(), n * 4, cudaMemcpyHostToDevice));
    long long total = (long long)n * 4096;
    k1<<<(unsigned)((total + 255) / 256), 256>>>(dx, n, dout);
    CK(cudaDeviceSynchronize());
    std::vector<uint16_t> out(total);
    CK(cudaMemcpy(out.data(), dout, total * 2, cudaMemcpyDeviceToHost));
    FILE* f = fopen((dir + "/rs_probe1.bin").c_str(), "wb");
    fwrite(&n, 4, 1, f); fwrite(xs.data(), 4, n, f); fwrite(out.data(), 2, total, f); fclose(f);
    // random test
    int m = 1 << 20; std::vector<float> x2(m); std::vector<uint32_t> r2(m);
    uint64_t s = 88172645463325252ull;
    auto nx = [&]() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s; };
    for (int i = 0; i < m; ++i) { x2[i] = (float)((nx() >> 40) * (1.0 / 16777216.0) * 3.5); r2[i] = (uint32_t)nx(); }
    float* dx2; uint32_t* dr2; uint16_t* do2;
    CK(cudaMalloc(&dx2, m * 4)); CK(cudaMalloc(&dr2, m * 4)); CK(cudaMalloc(&do2, m * 2));
    CK(cudaMemcpy(dx2, x2.data(), m * 4, cudaMemcpyHostToDevice)); CK(cudaMemcpy(dr2, r2.data(), m * 4, cudaMemcpyHostToDevice));
    k2<<<(m + 255) / 256, 256>>>(dx2, dr2, m, do2);
    CK(cudaDeviceSynchronize());
    std::vector<uint16_t> o2(m);
    CK(cudaMemcpy(o2.data(), do2, m * 2, cudaMemcpyDeviceToHost));
    f = fopen((dir + "/rs_probe2.bin").c_str(), "wb");
    fwrite(&m, 4, 1, f); fwrite(x2.data(), 4, m, f); fwrite(r2.data(), 4, m, f); fwrite(o2.data(), 2, m, f); fclose(f);
    printf("probe ok n=%d\n", n);
    return 0;
}
