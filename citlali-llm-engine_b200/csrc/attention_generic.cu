// The attention mixer's generic kernels: q/k head norm + rotation + cache write, and
// attention of every row over its slot's cached keys.  They take any head size up to 256,
// any number of heads and groups, any page size; they serve the true 32-bit path and are
// the bfloat16 path's kernels where the tensor-core ones refuse a shape.
#include "api.h"
#include "common.cuh"

namespace citlali {

constexpr int kMaxPairsPerLane = 4;   // head_dim <= 256: 128 rotation pairs over 32 lanes

// One warp per (row, head).  Heads 0..nq-1 are queries, then nkv key heads, then nkv value
// heads, as they lie in the fused projection's output row.
//   q, k: RMSNorm over the head with a gain shared by all heads (rms_norm_heads_kernel,
//         kernels.cu:95-124), then the half-split rotation by the row's position with
//         angle = float(pos) * inv_freq[i] (rope_kernel, kernels.cu:485-521; inv_freq[i] =
//         theta^(-2i/d) is tabulated by the host).  No rounding between the two.
//   k, v: stored at the row's position in the slot's pages (store_kv_kernel,
//         kernels.cu:524-533), k after norm and rotation, v as projected.
constexpr int kRopeWarps = 8;      // warps per block
constexpr int kMaxTailPerLane = 8; // head elements past the rotated ones: at most 254 over 32 lanes

// `write_cache`: 0 nothing is stored to the cache (a layer that reads another layer's keys); 1 keys and
// values go to the cache; 2 the normed (and rotated) keys go back into the row instead and values stay
// where they are, for a position encoding that works on the row between this kernel and the cache write.
// PARTIAL: only the first `rotary_dim` elements of a head are rotated, in pairs (i, i + rotary_dim/2);
// the rest are normed and pass through.
template <typename T, typename TG, bool PARTIAL>
__global__ void __launch_bounds__(kRopeWarps * 32)
qk_norm_rope_cache_kernel(T* __restrict__ qkv, const TG* __restrict__ q_gain, const TG* __restrict__ k_gain,
                          const float* __restrict__ inv_freq, int rotary_dim,
                          const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                          const int32_t* __restrict__ page_table, int page_table_stride,
                          T* __restrict__ k_pool, T* __restrict__ v_pool, int page_size,
                          int nq, int nkv, int d, float eps, int write_cache, int heads_per_block) {
    extern __shared__ float2 cos_sin[];                 // [rotary_dim / 2]: the row's rotation, shared by the block's heads
    dependents_may_launch();
    // positions, slots and page tables come from the host before the step: the rotation and the row's place in
    // the cache are worked out while the kernel ahead (the projection) is still running
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int total = nq + 2 * nkv;
    const int head_begin = blockIdx.y * heads_per_block;
    const int head_end = min(total, head_begin + heads_per_block);
    const int half = d >> 1;
    const int rh = PARTIAL ? (rotary_dim >> 1) : half;  // pairs that are rotated, and the distance within a pair
    const int pos = row_pos[row];
    for (int i = threadIdx.x; i < rh; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        cos_sin[i] = make_float2(cs, sn);
    }
    size_t page_off = 0;
    if (write_cache == 1) {
        const int page = page_table[(size_t)row_slot[row] * page_table_stride + pos / page_size];
        page_off = ((size_t)page * nkv * page_size + (pos % page_size)) * d;       // + kv head * page_size * d
    }
    __syncthreads();
    wait_for_predecessor();
    T* row_ptr = qkv + (size_t)row * total * d;

    // a warp takes heads warp, warp + 8, ...
    for (int head = head_begin + warp; head < head_end; head += kRopeWarps) {
        const bool is_v = head >= nq + nkv;
        // a value head is copied as two halves; a query or key head as its pairs and, if PARTIAL, its tail
        const int step = is_v ? half : rh;
        float x0[kMaxPairsPerLane], x1[kMaxPairsPerLane], tail[PARTIAL ? kMaxTailPerLane : 1];
#pragma unroll
        for (int j = 0; j < kMaxPairsPerLane; ++j) {
            const int i = lane + 32 * j;
            const bool on = i < step;
            x0[j] = on ? ldf(row_ptr, (size_t)head * d + i) : 0.0f;
            x1[j] = on ? ldf(row_ptr, (size_t)head * d + i + step) : 0.0f;
        }
        if (PARTIAL) {
#pragma unroll
            for (int j = 0; j < kMaxTailPerLane; ++j) {
                const int i = 2 * rh + lane + 32 * j;
                tail[j] = (!is_v && i < d) ? ldf(row_ptr, (size_t)head * d + i) : 0.0f;
            }
        }
        if (is_v) {                                     // a value head goes to the cache as it is
            if (write_cache == 1) {
                T* dst = v_pool + page_off + (size_t)((head - nq) % nkv) * page_size * d;
#pragma unroll
                for (int j = 0; j < kMaxPairsPerLane; ++j) {
                    const int i = lane + 32 * j;
                    if (i < half) { stf(dst, i, x0[j]); stf(dst, i + half, x1[j]); }
                }
            }
            continue;
        }
        const bool is_q = head < nq;
        const TG* gain = is_q ? q_gain : k_gain;
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < kMaxPairsPerLane; ++j) {
            ss = fmaf(x0[j], x0[j], ss);
            ss = fmaf(x1[j], x1[j], ss);
        }
        if (PARTIAL) {
#pragma unroll
            for (int j = 0; j < kMaxTailPerLane; ++j) ss = fmaf(tail[j], tail[j], ss);
        }
        ss = warp_sum(ss);
        const float inv = gain ? rsqrtf(ss / (float)d + eps) : 1.0f;
        if (!is_q && write_cache == 0) continue;
        T* dst = (is_q || write_cache == 2) ? row_ptr + (size_t)head * d
                                            : k_pool + page_off + (size_t)((head - nq) % nkv) * page_size * d;
#pragma unroll
        for (int j = 0; j < kMaxPairsPerLane; ++j) {
            const int i = lane + 32 * j;
            if (i < rh) {
                float a = x0[j], c2 = x1[j];
                if (gain) {
                    a = a * inv * ldf(gain, i);
                    c2 = c2 * inv * ldf(gain, i + rh);
                }
                const float c = cos_sin[i].x, sn = cos_sin[i].y;
                stf(dst, i, a * c - c2 * sn);
                stf(dst, i + rh, a * sn + c2 * c);
            }
        }
        if (PARTIAL) {
#pragma unroll
            for (int j = 0; j < kMaxTailPerLane; ++j) {
                const int i = 2 * rh + lane + 32 * j;
                if (i < d) stf(dst, i, gain ? tail[j] * inv * ldf(gain, i) : tail[j]);
            }
        }
    }
}

// The same for bfloat16 rows whose half head is a power-of-two number of 16-byte pieces (head sizes
// 16, 32, 64, 128, 256): `lanes` = head_dim / 16 neighbouring lanes share a head, each with eight
// elements of the first half and the eight they pair with in the second, moved as 16-byte words.
constexpr int kRopeVecThreads = 128;

__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 w;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return w;
}

template <typename TG>
__global__ void __launch_bounds__(kRopeVecThreads)
qk_norm_rope_cache_vec_kernel(__nv_bfloat16* __restrict__ qkv, const TG* __restrict__ q_gain, const TG* __restrict__ k_gain,
                              const float* __restrict__ inv_freq,
                              const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                              const int32_t* __restrict__ page_table, int page_table_stride,
                              __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, int page_size,
                              int nq, int nkv, int d, float eps, int write_cache, int heads_per_block, int lanes) {
    extern __shared__ float2 cos_sin[];                 // [d / 2]: the row's rotation, shared by the block's heads
    dependents_may_launch();
    // (as above: everything that does not come from the projection is done before waiting for it)
    const int row = blockIdx.x;
    const int total = nq + 2 * nkv;
    const int head_begin = blockIdx.y * heads_per_block;
    const int head_end = min(total, head_begin + heads_per_block);
    const int half = d >> 1;
    const int pos = row_pos[row];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        cos_sin[i] = make_float2(cs, sn);
    }
    size_t page_off = 0;
    if (write_cache) {
        const int page = page_table[(size_t)row_slot[row] * page_table_stride + pos / page_size];
        page_off = ((size_t)page * nkv * page_size + (pos % page_size)) * d;       // + kv head * page_size * d
    }
    __syncthreads();
    wait_for_predecessor();
    __nv_bfloat16* row_ptr = qkv + (size_t)row * total * d;
    const int part = threadIdx.x % lanes, e0 = part * 8;      // this lane's elements e0..e0+7 of each half
    const int heads_per_pass = kRopeVecThreads / lanes;
    for (int h0 = head_begin; h0 < head_end; h0 += heads_per_pass) {      // the same trip count for every lane
        const int head = h0 + threadIdx.x / lanes;
        const bool on = head < head_end;
        float x0[8], x1[8];
        if (on) {
            unpack8(*reinterpret_cast<const uint4*>(row_ptr + (size_t)head * d + e0), x0);
            unpack8(*reinterpret_cast<const uint4*>(row_ptr + (size_t)head * d + half + e0), x1);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) x0[i] = x1[i] = 0.0f;
        }
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) { ss = fmaf(x0[i], x0[i], ss); ss = fmaf(x1[i], x1[i], ss); }
        for (int o = lanes >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (!on) continue;
        if (head >= nq + nkv) {                         // a value head goes to the cache as it is
            if (write_cache) {
                __nv_bfloat16* dst = v_pool + page_off + (size_t)((head - nq) % nkv) * page_size * d;
                *reinterpret_cast<uint4*>(dst + e0) = pack8(x0);
                *reinterpret_cast<uint4*>(dst + half + e0) = pack8(x1);
            }
            continue;
        }
        const bool is_q = head < nq;
        if (!is_q && !write_cache) continue;
        const TG* gain = is_q ? q_gain : k_gain;
        if (gain) {
            const float inv = rsqrtf(ss / (float)d + eps);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                x0[i] = x0[i] * inv * ldf(gain, e0 + i);
                x1[i] = x1[i] * inv * ldf(gain, half + e0 + i);
            }
        }
        float y0[8], y1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 cs = cos_sin[e0 + i];
            y0[i] = x0[i] * cs.x - x1[i] * cs.y;
            y1[i] = x0[i] * cs.y + x1[i] * cs.x;
        }
        __nv_bfloat16* dst = is_q ? row_ptr + (size_t)head * d : k_pool + page_off + (size_t)((head - nq) % nkv) * page_size * d;
        *reinterpret_cast<uint4*>(dst + e0) = pack8(y0);
        *reinterpret_cast<uint4*>(dst + half + e0) = pack8(y1);
    }
}

// One block per (row, query head).  Query head j reads KV head j / (nq / nkv)
// (attention_scores_kernel, kernels.cu:564-565).  Keys lo..pos of the row's slot:
//   s_t = (q . k_t) * scale;  m = max s_t;  e_t = exp(s_t - m);  Z = sum e_t;
//   o_i = sum_t (e_t / Z) v_t[i]   with the division per term, t ascending
// (attention_values_kernel, kernels.cu:605-649).  Every reduction's order is a function of
// the number of keys alone, so a row's result does not depend on the step it came in.
template <typename T>
__global__ void __launch_bounds__(128)
attention_rows_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_pool,
                      const T* __restrict__ v_pool, const int32_t* __restrict__ page_table,
                      int page_table_stride, const int32_t* __restrict__ row_slot,
                      const int32_t* __restrict__ row_pos, T* __restrict__ out, int out_stride,
                      int nq, int nkv, int d, int page_size, int window, float scale) {
    extern __shared__ float smem[];
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = head / (nq / nkv);
    const int pos = row_pos[row];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n = pos - lo + 1;
    float* qs = smem;          // d
    float* sc = smem + d;      // n
    const int32_t* pages = page_table + (size_t)row_slot[row] * page_table_stride;

    const T* qrow = q + (size_t)row * q_stride + (size_t)head * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) qs[i] = ldf(qrow, i);
    __syncthreads();

    for (int t = warp; t < n; t += 4) {
        const int key = lo + t;
        const T* krow = k_pool + (((size_t)pages[key / page_size] * nkv + g) * page_size + key % page_size) * d;
        float s = 0.0f;
        for (int i = lane; i < d; i += 32) s = fmaf(qs[i], ldf(krow, i), s);
        s = warp_sum(s);
        if (lane == 0) sc[t] = s * scale;
    }
    __syncthreads();

    float m = -INFINITY;
    for (int t = threadIdx.x; t < n; t += blockDim.x) m = fmaxf(m, sc[t]);
    m = block_max(m, scratch);
    float z = 0.0f;
    for (int t = threadIdx.x; t < n; t += blockDim.x) {
        const float e = expf(sc[t] - m);
        sc[t] = e;
        z += e;
    }
    z = block_sum(z, scratch);
    for (int t = threadIdx.x; t < n; t += blockDim.x) sc[t] = sc[t] / z;
    __syncthreads();

    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.0f;
        for (int t = 0; t < n; ++t) {
            const int key = lo + t;
            const T* vrow = v_pool + (((size_t)pages[key / page_size] * nkv + g) * page_size + key % page_size) * d;
            acc = fmaf(sc[t], ldf(vrow, i), acc);
        }
        stf(out, (size_t)row * out_stride + (size_t)head * d + i, acc);
    }
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_qk_norm_rope_cache(void* qkv, int dtype, const void* q_gain, const void* k_gain, int gain_dtype,
                                          const float* inv_freq, int rotary_dim,
                                          const int32_t* row_slot, const int32_t* row_pos,
                                          const int32_t* page_table, int page_table_stride,
                                          void* k_pool, void* v_pool, int cache_dtype, int page_size,
                                          int rows, int nq, int nkv, int head_dim, float eps, int write_cache,
                                          cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (head_dim <= 0 || head_dim % 2 != 0 || head_dim > 64 * kMaxPairsPerLane) {
        set_last_error("qk_norm_rope_cache: head size %d must be even and at most %d", head_dim, 64 * kMaxPairsPerLane);
        return kBadShape;
    }
    if (rotary_dim <= 0 || rotary_dim % 2 != 0 || rotary_dim > head_dim) {
        set_last_error("qk_norm_rope_cache: the rotated part of a head (%d elements) must be even and at most the head size %d",
                       rotary_dim, head_dim);
        return kBadShape;
    }
    if (write_cache < 0 || write_cache > 2) {
        set_last_error("qk_norm_rope_cache: write_cache must be 0 (nothing), 1 (to the cache) or 2 (keys back into the row), not %d",
                       write_cache);
        return kBadShape;
    }
    const bool partial = rotary_dim != head_dim;
    if (cache_dtype != dtype) {
        set_last_error("qk_norm_rope_cache: the cache's dtype must equal the activations'");
        return kBadDType;
    }
    if (nq <= 0 || nkv < 0 || page_size <= 0) {
        set_last_error("qk_norm_rope_cache: bad head counts (%d, %d) or page size %d", nq, nkv, page_size);
        return kBadShape;
    }
    const int total = nq + 2 * nkv;
    // many rows (prompts): one block rotates all heads of a row from one table; few rows (decoding):
    // eight heads a block, so that there are enough blocks
    const int heads_per_block = rows >= 128 ? total : kRopeWarps;
    dim3 grid(rows, (total + heads_per_block - 1) / heads_per_block);
    if (grid.y > 65535) {
        set_last_error("qk_norm_rope_cache: too many heads (%d)", total);
        return kTooLarge;
    }
    // bfloat16 with a power-of-two number of 16-byte pieces in half a head: the kernel that moves 16-byte words
    const int lanes = head_dim / 16;
    if (!partial && write_cache != 2 && dtype == kBF16 && head_dim % 16 == 0 && (lanes & (lanes - 1)) == 0 && lanes <= 32 &&
        ((uintptr_t)qkv & 15u) == 0 && ((uintptr_t)k_pool & 15u) == 0 && ((uintptr_t)v_pool & 15u) == 0) {
        const int per_pass = kRopeVecThreads / lanes;
        const int vec_heads = rows >= 128 ? total : per_pass;
        dim3 vec_grid(rows, (total + vec_heads - 1) / vec_heads);
        return CITLALI_DISPATCH_FLOAT(gain_dtype, TG, [&] {
            launch_kernel(qk_norm_rope_cache_vec_kernel<TG>, vec_grid, kRopeVecThreads, (size_t)(head_dim / 2) * sizeof(float2), stream,
                (__nv_bfloat16*)qkv, (const TG*)q_gain, (const TG*)k_gain, inv_freq, row_slot, row_pos, page_table,
                page_table_stride, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, page_size, nq, nkv, head_dim, eps, write_cache,
                vec_heads, lanes);
            return CITLALI_LAUNCH_CHECK();
        });
    }
    return CITLALI_DISPATCH_FLOAT(dtype, T, [&] {
        return CITLALI_DISPATCH_FLOAT(gain_dtype, TG, [&] {
            if (partial) {
                launch_kernel(qk_norm_rope_cache_kernel<T, TG, true>, grid, kRopeWarps * 32, (size_t)(rotary_dim / 2) * sizeof(float2), stream,
                    (T*)qkv, (const TG*)q_gain, (const TG*)k_gain, inv_freq, rotary_dim, row_slot, row_pos, page_table,
                    page_table_stride, (T*)k_pool, (T*)v_pool, page_size, nq, nkv, head_dim, eps, write_cache, heads_per_block);
            } else {
                launch_kernel(qk_norm_rope_cache_kernel<T, TG, false>, grid, kRopeWarps * 32, (size_t)(head_dim / 2) * sizeof(float2), stream,
                    (T*)qkv, (const TG*)q_gain, (const TG*)k_gain, inv_freq, rotary_dim, row_slot, row_pos, page_table,
                    page_table_stride, (T*)k_pool, (T*)v_pool, page_size, nq, nkv, head_dim, eps, write_cache, heads_per_block);
            }
            return CITLALI_LAUNCH_CHECK();
        });
    });
}

extern "C" int citlali_attention_rows(const void* q, int q_stride, int dtype,
                                      const void* k_pool, const void* v_pool, int cache_dtype,
                                      const int32_t* page_table, int page_table_stride,
                                      const int32_t* row_slot, const int32_t* row_pos,
                                      void* out, int out_stride, int rows, int nq, int nkv, int head_dim,
                                      int page_size, int window, int max_keys, float scale,
                                      cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (cache_dtype != dtype) {
        set_last_error("attention_rows: the cache's dtype must equal the activations'");
        return kBadDType;
    }
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || head_dim <= 0 || nq > 65535) {
        set_last_error("attention_rows: %d query heads do not group over %d key/value heads (head size %d)",
                       nq, nkv, head_dim);
        return kBadShape;
    }
    const size_t smem = (size_t)(head_dim + max_keys) * sizeof(float);
    if (smem > 200 * 1024) {
        set_last_error("attention_rows: %d keys for one row need %zu bytes of shared memory, more than 204800",
                       max_keys, smem);
        return kTooLarge;
    }
    return CITLALI_DISPATCH_FLOAT(dtype, T, [&] {
        auto kernel = attention_rows_kernel<T>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        dim3 grid(rows, nq);
        launch_kernel(kernel, grid, 128, smem, stream, (const T*)q, q_stride, (const T*)k_pool, (const T*)v_pool, page_table,
                                             page_table_stride, row_slot, row_pos, (T*)out, out_stride, nq, nkv,
                                             head_dim, page_size, window, scale);
        return CITLALI_LAUNCH_CHECK();
    });
}
