// Choosing a token from float32 logits on the device: argmax and temperature sampling.
//
// The reference copies the logits to the host and scans them there: index order, non-finite
// values skipped, strict '>' so that the lowest index wins a tie, id 0 if nothing is finite
// (sample_greedy_from_logits, src/model/qwen_model.cpp:448-465).  argmax_rows keeps those
// rules.  Temperature sampling has no counterpart there.
#include "api.h"
#include "common.cuh"

namespace citlali {

__device__ __forceinline__ bool is_finite(float v) { return fabsf(v) <= 3.402823466e+38f; }

__device__ __forceinline__ void better(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// Block-wide (value, index) argmax over finite entries; all threads get the result.
__device__ void block_argmax(const float* __restrict__ row, int vocab, float& best, int& best_id,
                             float* sv, int* si) {
    float v = -INFINITY;
    int id = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = row[i];
        if (is_finite(x) && x > v) { v = x; id = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, id, o);
        better(v, id, ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = id; }
    __syncthreads();
    v = lane < nwarps ? sv[lane] : -INFINITY;
    id = lane < nwarps ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, id, o);
        better(v, id, ov, oi);
    }
    best = v;
    best_id = (id == 0x7fffffff) ? 0 : id;
}

__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const float* __restrict__ logits, int32_t* __restrict__ tokens, int vocab) {
    __shared__ float sv[32];
    __shared__ int si[32];
    dependents_may_launch();
    wait_for_predecessor();
    float best;
    int best_id;
    block_argmax(logits + (size_t)blockIdx.x * vocab, vocab, best, best_id, sv, si);
    if (threadIdx.x == 0) tokens[blockIdx.x] = best_id;
}

// The same in two steps for large vocabularies: each block scans one segment of a row, then one
// small block per row picks among the segments (lowest index on ties, as in a single scan).
constexpr int kArgmaxSegments = 64;

__global__ void __launch_bounds__(256)
argmax_segments_kernel(const float* __restrict__ logits, float* __restrict__ seg_value, int* __restrict__ seg_index, int vocab) {
    __shared__ float sv[32];
    __shared__ int si[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.y, seg = blockIdx.x;
    const int len = (vocab + kArgmaxSegments - 1) / kArgmaxSegments;
    const int begin = seg * len, end = min(vocab, begin + len);
    float best = -INFINITY;
    int best_id = 0;
    if (begin < end) {
        block_argmax(logits + (size_t)row * vocab + begin, end - begin, best, best_id, sv, si);
        best_id = best == -INFINITY ? 0x7fffffff : best_id + begin;
    } else {
        best_id = 0x7fffffff;
    }
    if (threadIdx.x == 0) {
        seg_value[row * kArgmaxSegments + seg] = best;
        seg_index[row * kArgmaxSegments + seg] = best_id;
    }
}

__global__ void __launch_bounds__(kArgmaxSegments)
argmax_pick_kernel(const float* __restrict__ seg_value, const int* __restrict__ seg_index, int32_t* __restrict__ tokens) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    float v = seg_value[row * kArgmaxSegments + threadIdx.x];
    int id = seg_index[row * kArgmaxSegments + threadIdx.x];
    if (v == -INFINITY) id = 0x7fffffff;
    __shared__ float sv[2];
    __shared__ int si[2];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, id, o);
        better(v, id, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = v; si[threadIdx.x >> 5] = id; }
    __syncthreads();
    if (threadIdx.x == 0) {
        better(v, id, sv[1], si[1]);
        tokens[row] = id == 0x7fffffff ? 0 : id;
    }
}

// p = softmax(logits / temperature) over finite entries; the token is the first index whose
// inclusive CDF, accumulated in index order, exceeds u.  The vocabulary is cut into 32
// contiguous segments, one per warp; segment sums locate the segment, then one warp walks it
// 32 entries at a time with an inclusive scan.  Every order is fixed by the vocabulary size.
__global__ void __launch_bounds__(1024)
sample_rows_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                   const float* __restrict__ uniform, int32_t* __restrict__ tokens, int vocab) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float seg_sum[32];
    dependents_may_launch();
    wait_for_predecessor();
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const float temp = temperature[blockIdx.x];
    float best;
    int best_id;
    block_argmax(row, vocab, best, best_id, sv, si);
    if (!(temp > 0.0f) || best == -INFINITY) {
        if (threadIdx.x == 0) tokens[blockIdx.x] = best_id;
        return;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seg = ((vocab + 1023) / 1024) * 32;        // segment length, a multiple of 32
    const float inv_t = 1.0f / temp;
    {
        float s = 0.0f;
        const int begin = warp * seg, end = min(vocab, begin + seg);
        for (int i = begin + lane; i < end; i += 32) {
            const float x = row[i];
            if (is_finite(x)) s += expf((x - best) * inv_t);
        }
        s = warp_sum(s);
        if (lane == 0) seg_sum[warp] = s;
    }
    __syncthreads();
    if (warp != 0) return;
    float total = 0.0f;
    for (int w = 0; w < 32; ++w) total += seg_sum[w];
    const float target = uniform[blockIdx.x] * total;
    float running = 0.0f;
    int w0 = 0;
    while (w0 < 31 && running + seg_sum[w0] <= target) { running += seg_sum[w0]; ++w0; }
    int chosen = -1, last_mass = best_id;
    for (int base = w0 * seg; base < vocab && chosen < 0; base += 32) {
        const int i = base + lane;
        float e = 0.0f;
        if (i < vocab) {
            const float x = row[i];
            if (is_finite(x)) e = expf((x - best) * inv_t);
        }
        float scan = e;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, scan, o);
            if (lane >= o) scan += up;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, e > 0.0f && running + scan > target);
        const unsigned mass = __ballot_sync(0xffffffffu, e > 0.0f);
        if (hit) chosen = base + __ffs(hit) - 1;
        if (mass) last_mass = base + 31 - __clz(mass);
        running += __shfl_sync(0xffffffffu, scan, 31);
    }
    if (lane == 0) tokens[blockIdx.x] = chosen >= 0 ? chosen : last_mass;
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_argmax_rows(const float* logits, int32_t* tokens, int rows, int vocab, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) {
        set_last_error("argmax_rows: vocabulary size %d must be positive", vocab);
        return kBadShape;
    }
    launch_kernel(argmax_rows_kernel, rows, 1024, 0, stream, logits, tokens, vocab);
    return CITLALI_LAUNCH_CHECK();
}

// The same with `scratch` (rows * 128 floats, 4-byte aligned): the vocabulary of every row is
// scanned by 64 blocks.  Worth it from a few thousand entries on.
extern "C" int citlali_argmax_rows_wide(const float* logits, int32_t* tokens, float* scratch, int rows, int vocab,
                                        cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || rows > 65535 || scratch == nullptr) {
        set_last_error("argmax_rows_wide: vocabulary %d must be positive, rows %d at most 65535, scratch given", vocab, rows);
        return kBadShape;
    }
    float* seg_value = scratch;
    int* seg_index = reinterpret_cast<int*>(scratch + (size_t)rows * kArgmaxSegments);
    launch_kernel(argmax_segments_kernel, dim3(kArgmaxSegments, rows), 256, 0, stream, logits, seg_value, seg_index, vocab);
    launch_kernel(argmax_pick_kernel, rows, kArgmaxSegments, 0, stream, (const float*)seg_value, (const int*)seg_index, tokens);
    return CITLALI_LAUNCH_CHECK();
}

extern "C" int citlali_sample_rows(const float* logits, const float* temperature, const float* uniform,
                                   int32_t* tokens, int rows, int vocab, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) {
        set_last_error("sample_rows: vocabulary size %d must be positive", vocab);
        return kBadShape;
    }
    launch_kernel(sample_rows_kernel, rows, 1024, 0, stream, logits, temperature, uniform, tokens, vocab);
    return CITLALI_LAUNCH_CHECK();
}
