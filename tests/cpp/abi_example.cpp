// A C++ program that uses the kernel library through its C interface alone (csrc/api.h): an RMSNorm, a float32 product
// and the tensor-core product with its bounded waits' fault word, checked against sums made here on the host.
// Built and run by tests/test_gpu_cpp_abi.py; prints "ok" and exits 0, or says what differed and exits 1.
#include "api.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#define CHECK_CUDA(call)                                                                        \
    do {                                                                                        \
        cudaError_t e_ = (call);                                                                \
        if (e_ != cudaSuccess) { std::printf("%s: %s\n", #call, cudaGetErrorString(e_)); return 1; } \
    } while (0)
#define CHECK_LIB(call)                                                                         \
    do {                                                                                        \
        int r_ = (call);                                                                        \
        if (r_ != 0) { std::printf("%s returned %d: %s\n", #call, r_, citlali_last_error()); return 1; } \
    } while (0)

static float uniform(unsigned& state) {
    state = state * 1664525u + 1013904223u;
    return (float)((state >> 8) & 0xFFFF) / 32768.0f - 1.0f;
}

int main() {
    const int rows = 5, hidden = 200, N = 48, K = 200;
    unsigned seed = 7;
    std::vector<float> x(rows * hidden), gain(hidden), w(N * K);
    for (float& v : x) v = uniform(seed) * 3.0f;
    for (float& v : gain) v = 1.0f + 0.2f * uniform(seed);
    for (float& v : w) v = uniform(seed) * 0.1f;
    float *dx, *dgain, *dh, *dw, *dy;
    CHECK_CUDA(cudaMalloc(&dx, x.size() * 4)); CHECK_CUDA(cudaMalloc(&dgain, gain.size() * 4));
    CHECK_CUDA(cudaMalloc(&dh, x.size() * 4)); CHECK_CUDA(cudaMalloc(&dw, w.size() * 4));
    CHECK_CUDA(cudaMalloc(&dy, rows * N * 4));
    CHECK_CUDA(cudaMemcpy(dx, x.data(), x.size() * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dgain, gain.data(), gain.size() * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dw, w.data(), w.size() * 4, cudaMemcpyHostToDevice));
    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));

    // h = rms_norm(x) * gain; y = h . w^T, all float32
    const float eps = 1e-5f;
    CHECK_LIB(citlali_rms_norm(dx, dgain, 0, nullptr, dh, 0, rows, hidden, eps, stream));
    CHECK_LIB(citlali_gemm_simt(dh, 0, dw, 0, dy, 0, rows, N, K, 0, stream));
    std::vector<float> y(rows * N);
    CHECK_CUDA(cudaMemcpyAsync(y.data(), dy, y.size() * 4, cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    double worst = 0.0, scale = 0.0;
    for (int r = 0; r < rows; ++r) {
        double ss = 0.0;
        for (int i = 0; i < hidden; ++i) ss += (double)x[r * hidden + i] * x[r * hidden + i];
        const double inv = 1.0 / std::sqrt(ss / hidden + eps);
        for (int n = 0; n < N; ++n) {
            double acc = 0.0;
            for (int k = 0; k < K; ++k) acc += x[r * hidden + k] * inv * gain[k] * w[n * K + k];
            worst = std::fmax(worst, std::fabs(acc - y[r * N + n]));
            scale = std::fmax(scale, std::fabs(acc));
        }
    }
    if (worst > 2e-5 * scale) { std::printf("float32 path: |diff| %.3e of %.3e\n", worst, scale); return 1; }

    // the tensor-core product: bfloat16 operands, float32 result, fault word untouched
    const int M2 = 8, N2 = 256, K2 = 512;
    std::vector<__nv_bfloat16> a(M2 * K2), b(N2 * K2);
    std::vector<float> af(a.size()), bf(b.size());
    for (size_t i = 0; i < a.size(); ++i) { a[i] = __float2bfloat16(uniform(seed)); af[i] = __bfloat162float(a[i]); }
    for (size_t i = 0; i < b.size(); ++i) { b[i] = __float2bfloat16(uniform(seed) * 0.1f); bf[i] = __bfloat162float(b[i]); }
    __nv_bfloat16 *da, *db;
    float* dc;
    int32_t* flag;
    CHECK_CUDA(cudaMalloc(&da, a.size() * 2)); CHECK_CUDA(cudaMalloc(&db, b.size() * 2));
    CHECK_CUDA(cudaMalloc(&dc, M2 * N2 * 4)); CHECK_CUDA(cudaMalloc(&flag, 16));
    CHECK_CUDA(cudaMemset(flag, 0, 16));
    CHECK_CUDA(cudaMemcpy(da, a.data(), a.size() * 2, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(db, b.data(), b.size() * 2, cudaMemcpyHostToDevice));
    CHECK_LIB(citlali_gemm_tc(da, db, dc, 0, M2, N2, K2, 0, 0, flag, 0, stream));
    std::vector<float> c(M2 * N2);
    int32_t words[4];
    CHECK_CUDA(cudaMemcpyAsync(c.data(), dc, c.size() * 4, cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaMemcpyAsync(words, flag, 16, cudaMemcpyDeviceToHost, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    worst = scale = 0.0;
    for (int m = 0; m < M2; ++m)
        for (int n = 0; n < N2; ++n) {
            double acc = 0.0;
            for (int k = 0; k < K2; ++k) acc += (double)af[m * K2 + k] * bf[n * K2 + k];
            worst = std::fmax(worst, std::fabs(acc - c[m * N2 + n]));
            scale = std::fmax(scale, std::fabs(acc));
        }
    if (worst > 1e-4 * scale) { std::printf("tensor-core product: |diff| %.3e of %.3e\n", worst, scale); return 1; }
    if (words[0] | words[1] | words[2] | words[3]) { std::printf("the fault word is %d %d %d %d\n", words[0], words[1], words[2], words[3]); return 1; }
    // a size the product does not take is refused with a message, nothing is launched
    if (citlali_gemm_tc(da, db, dc, 0, M2, N2, 20, 0, 0, flag, 0, stream) >= 0) { std::printf("K = 20 was not refused\n"); return 1; }
    std::printf("ok (%s)\n", citlali_last_error());
    return 0;
}
