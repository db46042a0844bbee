// y[M, N] = x[M, K] . w[N, K]^T on CUDA cores: float accumulation, k strictly ascending.
//
// This is the matrix product of the true 32-bit path, and the bfloat16 path's product for
// shapes the tensor-core kernel refuses.  One output element is one chain of fused
// multiply-adds over k = 0 .. K-1; the chain does not depend on M, on N, on where the
// element lies in a tile or on what else is in the batch, so a row's result is the same
// however the rows were cut into steps.  (The reference's product is one block per output
// row with a tree reduction, matvec_fp16_kernel, kernels.cu:381-449.)
#include "api.h"
#include "common.cuh"

namespace citlali {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16;

template <typename TX, typename TW, typename TY, bool kAccumulate>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y, int M, int N, int K) {
    __shared__ float xs[kTileK][kTileM + 4];
    __shared__ float ws[kTileK][kTileN + 4];
    dependents_may_launch();
    wait_for_predecessor();
    const int m0 = blockIdx.y * kTileM, n0 = blockIdx.x * kTileN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += kTileK) {
        // 64 rows x 16 k of each operand; 256 threads load 4 elements each, k fastest.
        for (int e = threadIdx.x; e < kTileM * kTileK; e += 256) {
            const int r = e / kTileK, kk = e % kTileK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            xs[kk][r] = (gm < M && gk < K) ? ldf(x, (size_t)gm * K + gk) : 0.0f;
            ws[kk][r] = (gn < N && gk < K) ? ldf(w, (size_t)gn * K + gk) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTileK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            const size_t o = (size_t)gm * N + gn;
            if (kAccumulate) stf(y, o, ldf(y, o) + acc[i][j]);
            else stf(y, o, acc[i][j]);
        }
    }
}

template <typename TX, typename TW, typename TY>
static int launch(const void* x, const void* w, void* y, int M, int N, int K, int accumulate, cudaStream_t stream) {
    dim3 grid((N + kTileN - 1) / kTileN, (M + kTileM - 1) / kTileM);
    if (grid.y > 65535) {
        set_last_error("gemm_simt: %d rows exceed the grid limit", M);
        return kTooLarge;
    }
    if (accumulate)
        launch_kernel(gemm_simt_kernel<TX, TW, TY, true>, grid, 256, 0, stream, (const TX*)x, (const TW*)w, (TY*)y, M, N, K);
    else
        launch_kernel(gemm_simt_kernel<TX, TW, TY, false>, grid, 256, 0, stream, (const TX*)x, (const TW*)w, (TY*)y, M, N, K);
    return CITLALI_LAUNCH_CHECK();
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype,
                                 int M, int N, int K, int accumulate, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) {
        set_last_error("gemm_simt: inner size %d must be positive", K);
        return kBadShape;
    }
    if (accumulate && y_dtype != kF32) {
        set_last_error("gemm_simt: accumulation needs a float32 output");
        return kBadDType;
    }
    return CITLALI_DISPATCH_FLOAT(x_dtype, TX, [&] {
        return CITLALI_DISPATCH_FLOAT(w_dtype, TW, [&] {
            return CITLALI_DISPATCH_FLOAT(y_dtype, TY, [&] {
                return launch<TX, TW, TY>(x, w, y, M, N, K, accumulate, stream);
            });
        });
    });
}
