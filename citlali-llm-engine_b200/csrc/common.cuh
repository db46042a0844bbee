// Shared device helpers: storage types, widening loads, rounding stores, block reductions.
//
// Every kernel widens what it reads to float, computes in float and rounds once at the
// store, as the reference's kernels do with half (src/compute/cuda/kernels.cu:13-24);
// storage here is bfloat16 or float.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace citlali {

enum DType : int { kF32 = 0, kBF16 = 1 };

// Error codes a launcher returns (0 = launched).  Negative values are refusals made on the
// host before any launch; positive values are cudaError_t.
enum Refusal : int {
    kOk = 0,
    kBadDType = -1,
    kBadShape = -2,
    kTooLarge = -3,
    kBadAlignment = -4,
    kNoDriverEntry = -5,
};

void set_last_error(const char* fmt, ...);

// ---- programmatic dependent launch -------------------------------------------------------
// Every kernel of the library is launched so that it may start while the kernel before it on
// the stream is still running.  The rule each kernel keeps: it says at once that its own
// successor may be launched (dependents_may_launch), and it does not read or write any global
// memory that other kernels write until the kernel before it has finished and its writes are
// visible (wait_for_predecessor).  What a kernel does before that wait must only touch memory
// that no kernel writes: weights.  Since a kernel cannot finish before its own wait has
// returned, everything older than the predecessor has finished as well.
__device__ __forceinline__ void dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool dependent_launch_enabled();

// The number of SMs of the current device, asked once per device.
inline int device_sm_count() {
    static int cached[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 1;
    if (cached[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 1;
        cached[device] = n;
    }
    return cached[device];
}

template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);     // errors surface in cudaGetLastError
}

// The same with the grid cut into clusters of `cluster_x` consecutive blocks (1: no clusters).
template <typename... KArgs, typename... Args>
inline void launch_kernel_clustered(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster_x,
                                    cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (dependent_launch_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float ldf(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void stf(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block whose size is a multiple of 32 (at most 1024); every thread gets the
// result.  `scratch` holds 32 floats.  The order of additions is fixed by the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.0f;
    return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
    return warp_max(t);
}

}  // namespace citlali

// Dispatch on a runtime dtype code to a template argument.
#define CITLALI_DISPATCH_FLOAT(code, T, ...)                                   \
    [&]() -> int {                                                             \
        if ((code) == citlali::kF32) { using T = float; return __VA_ARGS__(); }          \
        if ((code) == citlali::kBF16) { using T = __nv_bfloat16; return __VA_ARGS__(); } \
        citlali::set_last_error("dtype code %d is neither float32 (0) nor bfloat16 (1)", (int)(code)); \
        return (int)citlali::kBadDType;                                        \
    }()

#define CITLALI_LAUNCH_CHECK() (int)cudaGetLastError()
