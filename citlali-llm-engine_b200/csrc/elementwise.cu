// Row-wise kernels: embedding gather, RMSNorm, the SiLU gate.  One implementation serves
// the 32-bit path and the bfloat16 path; only storage types differ.
#include "api.h"
#include "common.cuh"

#include <cstdarg>
#include <cstdio>

namespace citlali {

static thread_local char g_last_error[512] = "";
static bool g_dependent_launch = true;

bool dependent_launch_enabled() { return g_dependent_launch; }

void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

// x = E[token] * scale; the reference copies the row with no scaling (embed_kernel, kernels.cu:27-35),
// which is scale = 1 (a product with 1.0f changes no bit).
// A token outside the vocabulary is not read: the row is zeroed and the flag is raised.
template <typename TW>
__global__ void embed_rows_kernel(const TW* __restrict__ table, const int32_t* __restrict__ tokens,
                                  float* __restrict__ out, int hidden, int vocab, float scale, int32_t* error_flag) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const int tok = tokens[row];
    const bool ok = tok >= 0 && tok < vocab;
    if (!ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
    const TW* src = table + (size_t)(ok ? tok : 0) * hidden;
    float* dst = out + (size_t)row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? ldf(src, i) * scale : 0.0f;
}

// What a layer norm that lives in the products around it needs of rows it has not seen come out of a product: the rows
// as bfloat16 and the sums of their squares over each 32 consecutive features (see citlali_gemm_tc_normed).  One block a
// row, one warp a group of 32 features at a time.
__global__ void norm_inputs_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ rows_out,
                                   float* __restrict__ sumsq, int hidden) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int groups = hidden >> 5;
    for (int g = warp; g < groups; g += warps) {
        const float v = x[(size_t)row * hidden + g * 32 + lane];
        rows_out[(size_t)row * hidden + g * 32 + lane] = __float2bfloat16_rn(v);
        const float sq = warp_sum(v * v);
        if (lane == 0) sumsq[(size_t)row * groups + g] = sq;
    }
}

// x *= scale over n floats (a logit scale; the reference has none).
__global__ void scale_kernel(float* __restrict__ x, size_t n, float scale) {
    dependents_may_launch();
    wait_for_predecessor();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] *= scale;
}

// inv = rsqrt(sum x^2 / n + eps); y = x * inv * gain (reference: rms_norm_kernel,
// kernels.cu:73-92, which runs one block per vector; here one block per row).
template <typename TG, typename TO>
__global__ void rms_norm_kernel(const float* __restrict__ x, const TG* __restrict__ gain,
                                const int32_t* __restrict__ row_index, TO* __restrict__ out,
                                int hidden, float eps) {
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const float* src = x + (size_t)(row_index ? row_index[row] : row) * hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = src[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    TO* dst = out + (size_t)row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) stf(dst, i, src[i] * inv * ldf(gain, i));
}

// The same for rows of at most 8192 elements that are a multiple of 4: every thread keeps its
// part of the row in registers, so the row is read once, with 16-byte loads.
template <typename TG, typename TO>
__global__ void __launch_bounds__(256)
rms_norm_rows_kernel(const float* __restrict__ x, const TG* __restrict__ gain,
                     const int32_t* __restrict__ row_index, TO* __restrict__ out, int hidden, float eps) {
    __shared__ float scratch[32];
    dependents_may_launch();
    // the gains (weights) and the row's index (from the host) are fetched while the kernel ahead still runs
    const int row = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(row_index ? row_index[row] : row) * hidden);
    const int quads = hidden >> 2;
    float4 g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int q = threadIdx.x + j * 256;
        g[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q < quads) {
            if constexpr (sizeof(TG) == 2) {
                const uint2 w = *reinterpret_cast<const uint2*>(gain + q * 4);
                const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.x));
                const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.y));
                g[j] = make_float4(lo.x, lo.y, hi.x, hi.y);
            } else {
                g[j] = *reinterpret_cast<const float4*>(gain + q * 4);
            }
        }
    }
    wait_for_predecessor();
    float4 v[8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int q = threadIdx.x + j * 256;
        v[j] = q < quads ? src[q] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    TO* dst = out + (size_t)row * hidden;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int q = threadIdx.x + j * 256;
        if (q < quads) {
            const int i = q * 4;
            const float a = v[j].x * inv * g[j].x, b = v[j].y * inv * g[j].y;
            const float c = v[j].z * inv * g[j].z, d = v[j].w * inv * g[j].w;
            if constexpr (sizeof(TO) == 2) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
                *reinterpret_cast<uint2*>(dst + i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            } else {
                *reinterpret_cast<float4*>(dst + i) = make_float4(a, b, c, d);
            }
        }
    }
}

// act = g / (1 + exp(-g)) * u (reference: swiglu_kernel, kernels.cu:474-482).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ act, int inter, int run) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const size_t base = (size_t)row * 2 * inter + (size_t)(i / run) * 2 * run + (i % run);
    const float g = ldf(gate_up, base);
    const float u = ldf(gate_up, base + run);
    stf(act, (size_t)row * inter + i, g / (1.0f + expf(-g)) * u);
}

}  // namespace citlali

using namespace citlali;

extern "C" const char* citlali_last_error(void) { return g_last_error; }

// 0: launch every kernel only after the one before it has finished; 1 (default): kernels may
// start early and wait on the device for their predecessor (programmatic dependent launch).
extern "C" void citlali_set_dependent_launch(int enabled) { g_dependent_launch = enabled != 0; }

extern "C" int citlali_embed_rows(const void* table, int table_dtype, const int32_t* tokens, float* out,
                                  int rows, int hidden, int vocab, float scale, int32_t* error_flag, cudaStream_t stream) {
    if (rows <= 0) return 0;
    return CITLALI_DISPATCH_FLOAT(table_dtype, TW, [&] {
        launch_kernel(embed_rows_kernel<TW>, rows, 256, 0, stream, (const TW*)table, tokens, out, hidden, vocab, scale, error_flag);
        return CITLALI_LAUNCH_CHECK();
    });
}

extern "C" int citlali_norm_inputs(const float* x, void* rows_out, float* sumsq, int rows, int hidden, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || hidden % 32 != 0) {
        set_last_error("norm_inputs: the width %d must be a multiple of 32", hidden);
        return kBadShape;
    }
    launch_kernel(norm_inputs_kernel, rows, hidden >= 2048 ? 512 : 128, 0, stream, x, (__nv_bfloat16*)rows_out, sumsq, hidden);
    return CITLALI_LAUNCH_CHECK();
}

extern "C" int citlali_scale(float* x, size_t n, float scale, cudaStream_t stream) {
    if (n == 0) return 0;
    const size_t blocks = (n + 255) / 256;
    launch_kernel(scale_kernel, (int)(blocks < 4096 ? blocks : 4096), 256, 0, stream, x, n, scale);
    return CITLALI_LAUNCH_CHECK();
}

extern "C" int citlali_rms_norm(const float* x, const void* gain, int gain_dtype, const int32_t* row_index,
                                void* out, int out_dtype, int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    return CITLALI_DISPATCH_FLOAT(gain_dtype, TG, [&] {
        return CITLALI_DISPATCH_FLOAT(out_dtype, TO, [&] {
            if (hidden % 4 == 0 && hidden <= 8192 && (((uintptr_t)gain | (uintptr_t)x | (uintptr_t)out) & 15u) == 0)
                launch_kernel(rms_norm_rows_kernel<TG, TO>, rows, 256, 0, stream, x, (const TG*)gain, row_index, (TO*)out, hidden, eps);
            else
                launch_kernel(rms_norm_kernel<TG, TO>, rows, threads, 0, stream, x, (const TG*)gain, row_index, (TO*)out, hidden, eps);
            return CITLALI_LAUNCH_CHECK();
        });
    });
}

extern "C" int citlali_swiglu(const void* gate_up, void* act, int dtype, int rows, int inter, int run,
                              cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (run <= 0 || inter % run != 0) {
        set_last_error("swiglu: gate/up run %d does not divide the intermediate size %d", run, inter);
        return kBadShape;
    }
    if ((inter + 255) / 256 > 65535) {
        set_last_error("swiglu: intermediate size %d exceeds the grid limit", inter);
        return kTooLarge;
    }
    return CITLALI_DISPATCH_FLOAT(dtype, T, [&] {
        dim3 grid(rows, (inter + 255) / 256);
        launch_kernel(swiglu_kernel<T>, grid, 256, 0, stream, (const T*)gate_up, (T*)act, inter, run);
        return CITLALI_LAUNCH_CHECK();
    });
}
