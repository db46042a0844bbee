// Attention of single new tokens over the paged cache, split over the context.
//
// A block takes (chunk of 256 keys = four pages, key/value head, sequence); its four warps take
// one page each.  The query heads that share the key/value head are processed together, so every
// key and value is read once for all of them.  Each warp keeps a running maximum, a running sum
// and a value accumulator (scores, maximum, exponentials and sums in float); the block merges its
// warps and writes one partial (m, l, acc) per head and chunk.  A second kernel merges the
// chunks in chunk order.  Positions come from device memory, so the launch does not depend on
// the sequences' lengths and the step can be replayed from a CUDA graph.
//
// The formulas are the reference's (attention_scores_kernel / attention_values_kernel,
// src/compute/cuda/kernels.cu:545-649): s = q.k / sqrt(d), softmax over keys lo..pos, weighted
// sum of values; query head j reads key/value head j / (heads / kv_heads).
#include "api.h"
#include "common.cuh"

namespace citlali {

constexpr int kChunkPages = 4;     // pages per block
constexpr int kDecodeWarps = 4;

// EPL consecutive bfloat16 of a key row and of a value row, widened to float, with one load each.
template <int EPL>
__device__ __forceinline__ void load_pair(const __nv_bfloat16* kp, const __nv_bfloat16* vp, float (&kf)[EPL], float (&vf)[EPL]) {
    if constexpr (EPL == 1) {
        kf[0] = __bfloat162float(*kp);
        vf[0] = __bfloat162float(*vp);
    } else {
        constexpr int kWords = EPL / 2;
        uint32_t kw[kWords], vw[kWords];
        if constexpr (EPL == 8) {
            const uint4 a = *reinterpret_cast<const uint4*>(kp), b = *reinterpret_cast<const uint4*>(vp);
            kw[0] = a.x; kw[1] = a.y; kw[2] = a.z; kw[3] = a.w; vw[0] = b.x; vw[1] = b.y; vw[2] = b.z; vw[3] = b.w;
        } else if constexpr (EPL == 4) {
            const uint2 a = *reinterpret_cast<const uint2*>(kp), b = *reinterpret_cast<const uint2*>(vp);
            kw[0] = a.x; kw[1] = a.y; vw[0] = b.x; vw[1] = b.y;
        } else {
            kw[0] = *reinterpret_cast<const uint32_t*>(kp);
            vw[0] = *reinterpret_cast<const uint32_t*>(vp);
        }
#pragma unroll
        for (int i = 0; i < kWords; ++i) {
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kw[i]));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vw[i]));
            kf[2 * i] = a.x; kf[2 * i + 1] = a.y; vf[2 * i] = b.x; vf[2 * i + 1] = b.y;
        }
    }
}

// EPL: elements of the head each lane owns (head_dim <= 32 * EPL); GT: query heads per block.
template <int EPL, int GT>
__global__ void __launch_bounds__(kDecodeWarps * 32)
attention_decode_partial_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                                const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                                const int32_t* __restrict__ page_table, int page_table_stride,
                                const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                                float* __restrict__ partial, int max_chunks,
                                int nq, int nkv, int d, int page_size, int window, float scale) {
    const int chunk = blockIdx.x;
    const int group = nq / nkv;
    const int tiles_per_kv = (group + GT - 1) / GT;
    const int g = blockIdx.y / tiles_per_kv;                   // key/value head
    const int head0 = g * group + (blockIdx.y % tiles_per_kv) * GT;   // first query head of this block
    const int heads_here = min(GT, g * group + group - head0);
    const int row = blockIdx.z;
    const int pos = row_pos[row];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int chunk_keys = kChunkPages * page_size;
    const int key0 = chunk * chunk_keys;
    if (key0 > pos || key0 + chunk_keys <= lo) return;        // nothing of this chunk is visible

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e0 = lane * EPL;
    const bool lane_on = e0 < d;
    const int32_t* pages = page_table + (size_t)row_slot[row] * page_table_stride;

    float qv[GT][EPL];
#pragma unroll
    for (int h = 0; h < GT; ++h)
#pragma unroll
        for (int e = 0; e < EPL; ++e)
            qv[h][e] = (lane_on && h < heads_here) ? __bfloat162float(q[(size_t)row * q_stride + (size_t)(head0 + h) * d + e0 + e]) * scale : 0.0f;

    float m[GT], l[GT], acc[GT][EPL];
#pragma unroll
    for (int h = 0; h < GT; ++h) {
        m[h] = -INFINITY; l[h] = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[h][e] = 0.0f;
    }

    const int page_index = chunk * kChunkPages + warp;
    const int first = max(page_index * page_size, lo);
    const int last = min(page_index * page_size + page_size - 1, pos);
    if (first <= last) {
        const size_t base = ((size_t)pages[page_index] * nkv + g) * page_size * d;
#pragma unroll 4
        for (int key = first; key <= last; ++key) {
            const size_t off = base + (size_t)(key - page_index * page_size) * d + e0;
            float kf[EPL], vf[EPL];
#pragma unroll
            for (int e = 0; e < EPL; ++e) { kf[e] = 0.0f; vf[e] = 0.0f; }
            if (lane_on) load_pair<EPL>(k_pool + off, v_pool + off, kf, vf);
            float s[GT];
#pragma unroll
            for (int h = 0; h < GT; ++h) {
                float t = 0.0f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) t = fmaf(qv[h][e], kf[e], t);
                s[h] = t;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int h = 0; h < GT; ++h) s[h] += __shfl_xor_sync(0xffffffffu, s[h], o);
#pragma unroll
            for (int h = 0; h < GT; ++h) {
                const float mn = fmaxf(m[h], s[h]);
                const float corr = __expf(m[h] - mn);          // exp(-inf) = 0 on the first key
                const float pw = __expf(s[h] - mn);
                l[h] = l[h] * corr + pw;
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[h][e] = fmaf(pw, vf[e], acc[h][e] * corr);
                m[h] = mn;
            }
        }
    }

    // merge the four warps: warp w parks (m, l, acc) in shared memory, warp 0 folds them in order
    extern __shared__ float park[];                             // [warps][GT][2 + 32 * EPL]
    const int per_head = 2 + 32 * EPL;
#pragma unroll
    for (int h = 0; h < GT; ++h) {
        float* slot = park + ((size_t)warp * GT + h) * per_head;
        if (lane == 0) { slot[0] = m[h]; slot[1] = l[h]; }
#pragma unroll
        for (int e = 0; e < EPL; ++e) slot[2 + e0 + e] = acc[h][e];
    }
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int h = 0; h < GT; ++h) {
        if (h >= heads_here) break;
        float M = -INFINITY;
        for (int w = 0; w < kDecodeWarps; ++w) M = fmaxf(M, park[((size_t)w * GT + h) * per_head]);
        float L = 0.0f, out[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) out[e] = 0.0f;
        for (int w = 0; w < kDecodeWarps; ++w) {
            const float* slot = park + ((size_t)w * GT + h) * per_head;
            const float f = (slot[0] == -INFINITY) ? 0.0f : __expf(slot[0] - M);
            L += slot[1] * f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) out[e] = fmaf(slot[2 + e0 + e], f, out[e]);
        }
        float* dst = partial + (((size_t)row * nq + head0 + h) * max_chunks + chunk) * (d + 2);
        if (lane == 0) { dst[0] = M; dst[1] = L; }
        if (lane_on) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) dst[2 + e0 + e] = out[e];
        }
    }
}

// out[row, head, :] = sum_c exp(m_c - M) acc_c / sum_c exp(m_c - M) l_c over the row's visible
// chunks, in chunk order.
__global__ void attention_decode_combine_kernel(const float* __restrict__ partial, int max_chunks,
                                                const int32_t* __restrict__ row_pos, __nv_bfloat16* __restrict__ out,
                                                int out_stride, int nq, int d, int chunk_keys, int window) {
    const int head = blockIdx.x, row = blockIdx.y;
    const int pos = row_pos[row];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int c0 = lo / chunk_keys, c1 = pos / chunk_keys;
    const float* base = partial + ((size_t)row * nq + head) * max_chunks * (d + 2);
    float M = -INFINITY;
    for (int c = c0; c <= c1; ++c) M = fmaxf(M, base[(size_t)c * (d + 2)]);
    float L = 0.0f;
    for (int c = c0; c <= c1; ++c) L += base[(size_t)c * (d + 2) + 1] * __expf(base[(size_t)c * (d + 2)] - M);
    const float inv = 1.0f / L;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float a = 0.0f;
        for (int c = c0; c <= c1; ++c) a = fmaf(base[(size_t)c * (d + 2) + 2 + i], __expf(base[(size_t)c * (d + 2)] - M), a);
        out[(size_t)row * out_stride + (size_t)head * d + i] = __float2bfloat16_rn(a * inv);
    }
}

template <int EPL, int GT>
static int launch_partial(const void* q, int q_stride, const void* k_pool, const void* v_pool, const int32_t* page_table,
                          int page_table_stride, const int32_t* row_slot, const int32_t* row_pos, float* partial,
                          int max_chunks, int rows, int nq, int nkv, int d, int page_size, int window, float scale,
                          cudaStream_t stream) {
    const int group = nq / nkv;
    const int tiles_per_kv = (group + GT - 1) / GT;
    dim3 grid(max_chunks, nkv * tiles_per_kv, rows);
    const size_t smem = (size_t)kDecodeWarps * GT * (2 + 32 * EPL) * sizeof(float);
    attention_decode_partial_kernel<EPL, GT><<<grid, kDecodeWarps * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, page_table,
        page_table_stride, row_slot, row_pos, partial, max_chunks, nq, nkv, d, page_size, window, scale);
    return CITLALI_LAUNCH_CHECK();
}

template <int EPL>
static int pick_gt(int gt, const void* q, int q_stride, const void* k_pool, const void* v_pool, const int32_t* page_table,
                   int page_table_stride, const int32_t* row_slot, const int32_t* row_pos, float* partial,
                   int max_chunks, int rows, int nq, int nkv, int d, int page_size, int window, float scale,
                   cudaStream_t stream) {
#define CITLALI_GT(G) return launch_partial<EPL, G>(q, q_stride, k_pool, v_pool, page_table, page_table_stride, row_slot, \
                                                     row_pos, partial, max_chunks, rows, nq, nkv, d, page_size, window, scale, stream)
    switch (gt) {
        case 1: CITLALI_GT(1);
        case 2: CITLALI_GT(2);
        case 4: CITLALI_GT(4);
        default: CITLALI_GT(8);
    }
#undef CITLALI_GT
}

}  // namespace citlali

using namespace citlali;

// Scratch for the partials of `rows` single-token rows whose positions stay below
// `max_positions`: floats.
extern "C" size_t citlali_attention_decode_scratch_floats(int rows, int nq, int head_dim, int page_size, int max_positions) {
    const int chunk_keys = kChunkPages * page_size;
    const int max_chunks = (max_positions + chunk_keys - 1) / chunk_keys;
    return (size_t)rows * nq * max_chunks * (head_dim + 2);
}

// Attention of `rows` single new tokens (bfloat16).  q rows are `q_stride` elements apart;
// positions and slots are read on the device; `max_positions` bounds the positions and fixes
// the grid.  `partial` holds citlali_attention_decode_scratch_floats(...) floats.
extern "C" int citlali_attention_decode(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                                        const int32_t* page_table, int page_table_stride,
                                        const int32_t* row_slot, const int32_t* row_pos,
                                        void* out, int out_stride, float* partial, size_t partial_floats,
                                        int rows, int nq, int nkv, int head_dim, int page_size, int window,
                                        int max_positions, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0) {
        set_last_error("attention_decode: %d query heads do not group over %d key/value heads", nq, nkv);
        return kBadShape;
    }
    if (head_dim <= 0 || head_dim % 8 != 0 || head_dim > 256) {
        set_last_error("attention_decode: head size %d must be a multiple of 8, at most 256", head_dim);
        return kBadShape;
    }
    if (rows > 65535 || nq > 65535) {
        set_last_error("attention_decode: %d rows or %d heads exceed the grid limit", rows, nq);
        return kTooLarge;
    }
    const int chunk_keys = kChunkPages * page_size;
    const int max_chunks = (max_positions + chunk_keys - 1) / chunk_keys;
    const size_t need = citlali_attention_decode_scratch_floats(rows, nq, head_dim, page_size, max_positions);
    if (partial == nullptr || partial_floats < need) {
        set_last_error("attention_decode: %zu floats of scratch are needed, %zu were given", need, partial_floats);
        return kTooLarge;
    }
    const int group = nq / nkv;
    const int gt = group <= 1 ? 1 : group <= 2 ? 2 : group <= 4 ? 4 : 8;
    int rc;
    // elements per lane: the smallest of 1, 2, 4, 8 that covers the head with 32 lanes and divides it
    int epl = head_dim <= 32 ? 1 : head_dim <= 64 ? 2 : head_dim <= 128 ? 4 : 8;
    while (head_dim % epl != 0) epl *= 2;   // cannot exceed 8 since head_dim % 8 == 0
#define CITLALI_EPL(E) rc = pick_gt<E>(gt, q, q_stride, k_pool, v_pool, page_table, page_table_stride, row_slot, row_pos, partial, \
                                        max_chunks, rows, nq, nkv, head_dim, page_size, window, scale, stream)
    switch (epl) {
        case 1: CITLALI_EPL(1); break;
        case 2: CITLALI_EPL(2); break;
        case 4: CITLALI_EPL(4); break;
        default: CITLALI_EPL(8); break;
    }
#undef CITLALI_EPL
    if (rc) return rc;
    dim3 grid(nq, rows);
    attention_decode_combine_kernel<<<grid, 128, 0, stream>>>(partial, max_chunks, row_pos, (__nv_bfloat16*)out, out_stride,
                                                              nq, head_dim, chunk_keys, window);
    return CITLALI_LAUNCH_CHECK();
}
