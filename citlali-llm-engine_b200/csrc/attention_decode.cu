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
#include "mma_common.cuh"

namespace citlali {

constexpr int kChunkPages = 4;     // pages per block of the CUDA-core kernel
constexpr int kKvStages = 3;       // key/value tiles in flight per block of the tensor-core kernel, plus the one in use
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
    dependents_may_launch();
    wait_for_predecessor();
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
        if (lane == 0) { dst[0] = M * 1.4426950408889634f; dst[1] = L; }   // maxima are stored in log2 units
        if (lane_on) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) dst[2 + e0 + e] = out[e];
        }
    }
}

// out[row, head, :] = sum_c 2^(m_c - M) acc_c / sum_c 2^(m_c - M) l_c over the row's visible
// chunks, in chunk order (m_c in log2 units).
__global__ void __launch_bounds__(128)
attention_decode_combine_kernel(const float* __restrict__ partial, int max_chunks,
                                const int32_t* __restrict__ row_pos, __nv_bfloat16* __restrict__ out,
                                int out_stride, int nq, int d, int chunk_keys, int window) {
    extern __shared__ float weight[];                           // [chunks]: 2^(m_c - M), then the total in [chunks]
    dependents_may_launch();
    wait_for_predecessor();
    const int head = blockIdx.x, row = blockIdx.y;
    const int pos = row_pos[row];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    // positions are below the launch's max_positions by contract (the host checks every step); a
    // position beyond it is clamped so that at least no partial is read that no block wrote
    const int c1 = min(pos / chunk_keys, max_chunks - 1);
    const int c0 = min(lo / chunk_keys, c1), n = c1 - c0 + 1;
    const float* base = partial + (((size_t)row * nq + head) * max_chunks + c0) * (d + 2);
    if (threadIdx.x < 32) {
        float M = -INFINITY;
        for (int c = threadIdx.x; c < n; c += 32) M = fmaxf(M, base[(size_t)c * (d + 2)]);
        M = warp_max(M);
        float L = 0.0f;
        for (int c = threadIdx.x; c < n; c += 32) {
            const float w = exp2f(base[(size_t)c * (d + 2)] - M);
            weight[c] = w;
            L += base[(size_t)c * (d + 2) + 1] * w;
        }
        L = warp_sum(L);
        if (threadIdx.x == 0) weight[n] = 1.0f / L;
    }
    __syncthreads();
    const float inv = weight[n];
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float a = 0.0f;
        for (int c = 0; c < n; ++c) a = fmaf(base[(size_t)c * (d + 2) + 2 + i], weight[c], a);
        out[(size_t)row * out_stride + (size_t)head * d + i] = __float2bfloat16_rn(a * inv);
    }
}

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// One float to shared-memory address `addr` of the block with rank `rank` in this cluster.
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// The same work on the tensor cores, for pages of 64 keys.  The rows of the MMA are the query
// heads that share the key/value head (padded to 16), so a key or value read from the cache
// serves all of them.  The block walks its chunk one page at a time (cp.async, double-buffered);
// each warp takes 16 keys of the page: S = Q K^T (mma.sync m16n8k16), online softmax in float,
// O += P V.  At the end the four warps' (m, l, O) are folded through shared memory (maxima in log2
// units), and the blocks of a cluster send their runs of a head to the block that merges that head.
constexpr int kMaxClusterBlocks = 16;     // blocks per (sequence, head group): a cluster, at most the non-portable size

// One head's (m, l, O) of `runs` consecutive runs of its keys ([run][D + 2] at `base`, m in log2 units), merged in run
// order into the head's output.  kFromL2: the runs were written by other blocks to global memory (read past L1).
template <int kBlocks, int D, bool kFromL2>
__device__ __forceinline__ void merge_runs(const float* base, int runs, __nv_bfloat16* out_head, int tid) {
    auto at = [&](size_t i) { return kFromL2 ? __ldcg(base + i) : base[i]; };
    float mz[kBlocks], wz[kBlocks];
#pragma unroll
    for (int z = 0; z < kBlocks; ++z) {
        mz[z] = z < runs ? at((size_t)z * (D + 2)) : -INFINITY;
        wz[z] = z < runs ? at((size_t)z * (D + 2) + 1) : 0.0f;           // l for now
    }
    float M = -INFINITY;
#pragma unroll
    for (int z = 0; z < kBlocks; ++z) M = fmaxf(M, mz[z]);
    float L = 0.0f;
#pragma unroll
    for (int z = 0; z < kBlocks; ++z) {
        const float f = mz[z] == -INFINITY ? 0.0f : exp2f(mz[z] - M);
        if (mz[z] != -INFINITY) L = fmaf(wz[z], f, L);
        wz[z] = f;
    }
    const float inv = 1.0f / L;
    for (int i = tid; i < D; i += 128) {
        float a = 0.0f;
#pragma unroll
        for (int z = 0; z < kBlocks; ++z)
            if (z < runs && mz[z] != -INFINITY) a = fmaf(at((size_t)z * (D + 2) + 2 + i), wz[z], a);
        out_head[i] = __float2bfloat16_rn(a * inv);
    }
}

// Block `rank` of a cluster merges heads rank, rank + split, ... over the (m, l, O) of all blocks' runs, which
// they have sent to `gathered` ([head / split][sender][D + 2]), in rank order.
template <int kBlocks, int D>
__device__ __forceinline__ void merge_gathered_heads(const float* gathered, __nv_bfloat16* out_row, int rank, int split, int heads_here, int tid) {
    for (int h = rank; h < heads_here; h += split)
        merge_runs<kBlocks, D, false>(gathered + (size_t)((h / split) * split) * (D + 2), split, out_row + (size_t)h * D, tid);
}

constexpr int kMaxRunsByLength = 8;      // blocks a row's keys are dealt to at most when the rows' lengths decide
constexpr int kMinRunTiles = 16;         // no run shorter than this many pages (measured: runs of 8 cost more than they balance)

//
// kByLength (many rows, no clusters; grid = head tiles x rows x runs, so that the blocks with nothing to do come
// last): the rows of a step can differ in length by an order of magnitude, and a block that walks the longest row
// alone is still walking when the others are done.  When the longest row has more than 1.3 times the mean number of
// pages, a row's pages are dealt to ceil(row's pages / (mean pages x run_scale_q8 / 256)) blocks, at most
// gridDim.z; a row's blocks write their (m, l, O) to `partial` ([row][head][run][D + 2]) and count themselves on
// counters[row, head tile]; the block that counts last merges the runs in run order and puts the counter back to
// zero.  Nobody waits for anybody.  Rows of about equal lengths keep one block each and nothing is merged.  The
// number of runs depends on the lengths in the step, which are read on the device: the launch does not.
//
// kPerWarp (one or few rows: a block an SM at most, clusters of up to sixteen): a warp does not take its 16 keys of
// every tile the block walks, with the block's two barriers a tile, but a run of 16-key units of its own, fetched into
// a ring of its own (kStagesKV units) and waited for by the warp alone.  Nothing in the loop holds a warp up for another.
template <int D, int kStagesKV, bool kByLength, bool kPerWarp = false>
__global__ void __launch_bounds__(128)
attention_decode_tc_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                           const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                           const int32_t* __restrict__ page_table, int page_table_stride,
                           const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                           __nv_bfloat16* __restrict__ out, int out_stride, int nq, int nkv, int window,
                           float scale_log2, float* __restrict__ partial, int* __restrict__ counters, int run_scale_q8) {
    using namespace fa;
    constexpr int kPage = 64;
    constexpr int kRowBytes = D * 2 + 16;
    constexpr int kTileBytes = kPage * kRowBytes;
    constexpr int kChunksPerRow = D / 8;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t s_q = (uint32_t)__cvta_generic_to_shared(smem);          // 16 rows
    const uint32_t s_k = s_q + 16 * kRowBytes, s_v = s_k + kStagesKV * kTileBytes;

    dependents_may_launch();
    int split = kByLength ? gridDim.z : gridDim.x;       // the blocks of a (sequence, head group) are one cluster
    const int rank = kByLength ? blockIdx.z : blockIdx.x;
    const int head_tile = kByLength ? blockIdx.x : blockIdx.y;
    const int group = nq / nkv;
    const int row_tiles = (group + 15) / 16;
    const int g = head_tile / row_tiles;
    const int head0 = g * group + (head_tile % row_tiles) * 16;
    const int heads_here = min(16, g * group + group - head0);
    const int row = kByLength ? blockIdx.y : blockIdx.z;
    const int pos = row_pos[row];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    // the visible pages are cut into `split` runs of equal length; this block takes run `rank` (it may be empty)
    const int first_page = lo / kPage, last_page = pos / kPage;
    if constexpr (kByLength) {
        // pages visible to all rows of the step (every warp adds them up for itself), their mean, this row's runs
        const int rows = gridDim.y;
        int total = 0, longest = 0;
        for (int r = threadIdx.x & 31; r < rows; r += 32) {
            const int p = row_pos[r];
            const int l = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
            const int pages = p / kPage - l / kPage + 1;
            total += pages;
            longest = max(longest, pages);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            total += __shfl_xor_sync(0xffffffffu, total, o);
            longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, o));
        }
        if ((long)longest * rows * 10 <= (long)total * 13) {
            split = 1;                                   // about equal lengths: a block a row
        } else {
            // run length: the mean times run_scale_q8 / 256, at least kMinRunTiles
            const long scaled = ((long)total * run_scale_q8 + (long)rows * 256 - 1) / ((long)rows * 256);
            const int run = scaled > kMinRunTiles ? (int)scaled : kMinRunTiles;
            const int mine = last_page - first_page + 1;
            split = min((int)gridDim.z, (mine + run - 1) / run);
        }
        if (rank >= split) return;
    }
    const int per_block = (last_page - first_page + split) / split;
    const int tile_lo = first_page + rank * per_block, tile_hi = min(tile_lo + per_block - 1, last_page);
    const int32_t* pages = page_table + (size_t)row_slot[row] * page_table_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;

    auto load_tile = [&](int tile, int buf) {
        const size_t base = ((size_t)pages[tile] * nkv + g) * kPage * D;
        for (int c = tid; c < kPage * kChunksPerRow; c += 128) {
            const int r = c / kChunksPerRow, ch = c % kChunksPerRow;
            const size_t src = base + (size_t)r * D + ch * 8;
            cp_async16(s_k + buf * kTileBytes + r * kRowBytes + ch * 16, k_pool + src);
            cp_async16(s_v + buf * kTileBytes + r * kRowBytes + ch * 16, v_pool + src);
        }
    };
    // Positions and page tables come from the host before the step, and every page but the row's last
    // holds keys and values of earlier steps only.  Unless the row's last page is among this block's
    // first tiles, they are fetched while the kernel ahead of this one (which writes the new token's
    // key, value and query) is still running.
    const bool early = tile_lo + kStagesKV - 2 < last_page;
    auto first_tiles = [&]() {
#pragma unroll
        for (int ahead = 0; ahead < kStagesKV - 1; ++ahead) {
            if (tile_lo + ahead <= tile_hi) load_tile(tile_lo + ahead, ahead);
            cp_async_commit();
        }
    };
    // kPerWarp: units of 16 keys; the visible units are cut into split * 4 runs of equal length, this warp takes run
    // rank * 4 + warp.  A unit's keys and values lie side by side in the warp's ring: [unit][keys | values].
    constexpr int kUnitBytes = 16 * kRowBytes;
    const int first_unit = lo >> 4, last_unit = pos >> 4;
    const int per_warp = (last_unit - first_unit + split * 4) / (split * 4);
    const int unit_lo = first_unit + (rank * 4 + warp) * per_warp, unit_hi = min(unit_lo + per_warp - 1, last_unit);
    const int my_units = unit_hi - unit_lo + 1;                      // may be zero or less
    const uint32_t ring = s_k + (uint32_t)warp * (kStagesKV * 2 * kUnitBytes);
    auto load_unit = [&](int unit, int slot) {
        const size_t base = (((size_t)pages[unit >> 2] * nkv + g) * kPage + (size_t)(unit & 3) * 16) * D;
        const uint32_t dst = ring + (uint32_t)slot * (2 * kUnitBytes);
        for (int c = lane; c < 16 * kChunksPerRow; c += 32) {
            const int r = c / kChunksPerRow, ch = c % kChunksPerRow;
            const size_t src = base + (size_t)r * D + ch * 8;
            cp_async16(dst + r * kRowBytes + ch * 16, k_pool + src);
            cp_async16(dst + kUnitBytes + r * kRowBytes + ch * 16, v_pool + src);
        }
    };
    if constexpr (kPerWarp) {
        // every unit but the row's last holds keys and values of earlier steps only: fetched before the kernel ahead
        // (which writes the new token's) has finished; the last unit, if it is among this warp's first, after it
#pragma unroll
        for (int i = 0; i < kStagesKV; ++i) {
            if (i < my_units && unit_lo + i != last_unit) load_unit(unit_lo + i, i);
            if (i < my_units && unit_lo + i == last_unit) break;    // its group is committed behind the wait, in order
            cp_async_commit();
        }
    } else if (early) {
        first_tiles();
    }
    wait_for_predecessor();
    if constexpr (kPerWarp) {
        if (unit_hi == last_unit && my_units >= 1 && my_units <= kStagesKV) {
            load_unit(last_unit, my_units - 1);
#pragma unroll 1
            for (int i = my_units - 1; i < kStagesKV; ++i) cp_async_commit();
        }
    }
    for (int c = tid; c < 16 * kChunksPerRow; c += 128) {
        const int r = c / kChunksPerRow, ch = c % kChunksPerRow;
        uint4 w = make_uint4(0, 0, 0, 0);
        if (r < heads_here) w = *reinterpret_cast<const uint4*>(q + (size_t)row * q_stride + (size_t)(head0 + r) * D + ch * 8);
        *reinterpret_cast<uint4*>(smem + r * kRowBytes + ch * 16) = w;
    }
    if (!kPerWarp && !early) first_tiles();

    uint32_t qf[D / 16][4];
    __syncthreads();
    {
        const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
        const int cbyte = (lane >> 4) * 16;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
            ldmatrix_x4(s_q + r * kRowBytes + ks * 32 + cbyte, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;

    const int steps = kPerWarp ? my_units : tile_hi - tile_lo + 1;
    for (int step = 0; step < steps; ++step) {
        const int tile = tile_lo + step;
        uint32_t kb, vb;
        if constexpr (kPerWarp) {
            cp_async_wait<kStagesKV - 1>();
            __syncwarp();
            kb = ring + (uint32_t)(step % kStagesKV) * (2 * kUnitBytes);
            vb = kb + kUnitBytes;
        } else {
            const int buf = step % kStagesKV;
            if (tile + kStagesKV - 1 <= tile_hi) load_tile(tile + kStagesKV - 1, (step + kStagesKV - 1) % kStagesKV);
            cp_async_commit();
            cp_async_wait<kStagesKV - 1>();
            __syncthreads();
            kb = s_k + buf * kTileBytes + warp * 16 * kRowBytes;
            vb = s_v + buf * kTileBytes + warp * 16 * kRowBytes;
        }
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int r = (lane & 7) + (lane >> 4) * 8;
            const int cbyte = ((lane >> 3) & 1) * 16;
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(kb + r * kRowBytes + ks * 32 + cbyte, b0, b1, b2, b3);
            mma_16816(s[0], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
            mma_16816(s[1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
        }
        const int key_base = (kPerWarp ? (unit_lo + step) * 16 : tile * kPage + warp * 16) + (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int key = key_base + i * 8;
            if (key > pos || key < lo) { s[i][0] = -INFINITY; s[i][2] = -INFINITY; }
            if (key + 1 > pos || key + 1 < lo) { s[i][1] = -INFINITY; s[i][3] = -INFINITY; }
        }
        float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float ref0 = mn0 == -INFINITY ? 0.0f : mn0 * scale_log2, ref1 = mn1 == -INFINITY ? 0.0f : mn1 * scale_log2;
        const float a0 = exp2f(m0 * scale_log2 - ref0), a1 = exp2f(m1 * scale_log2 - ref1);
        m0 = mn0; m1 = mn1;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            s[i][0] = exp2f(s[i][0] * scale_log2 - ref0); s[i][1] = exp2f(s[i][1] * scale_log2 - ref0);
            s[i][2] = exp2f(s[i][2] * scale_log2 - ref1); s[i][3] = exp2f(s[i][3] * scale_log2 - ref1);
        }
        l0 = l0 * a0 + s[0][0] + s[0][1] + s[1][0] + s[1][1];
        l1 = l1 * a1 + s[0][2] + s[0][3] + s[1][2] + s[1][3];
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
        const uint32_t p0 = pack_bf16(s[0][0], s[0][1]), p1 = pack_bf16(s[0][2], s[0][3]);
        const uint32_t p2 = pack_bf16(s[1][0], s[1][1]), p3 = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int np = 0; np < D / 16; ++np) {
            const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
            const int cbyte = np * 32 + (lane >> 4) * 16;
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(vb + r * kRowBytes + cbyte, b0, b1, b2, b3);
            mma_16816(o[2 * np], p0, p1, p2, p3, b0, b1);
            mma_16816(o[2 * np + 1], p0, p1, p2, p3, b2, b3);
        }
        if constexpr (kPerWarp) {
            __syncwarp();                                             // the slot is free: the unit a ring's length on
            if (step + kStagesKV < my_units) load_unit(unit_lo + step + kStagesKV, step % kStagesKV);
            cp_async_commit();
        } else {
            __syncthreads();
        }
    }
    cp_async_wait<0>();
    if constexpr (kPerWarp) __syncthreads();                          // the parked rows lie over the other warps' rings
    // This block no longer reads its tile buffers: it says so to the cluster at once and waits for the others
    // only before it writes into theirs.
    if (!kByLength && split > 1) cluster_arrive();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // park every warp's (m in log2 units, l, O) of the rows that hold heads over the tile buffers
    float* park = reinterpret_cast<float*>(smem + 16 * kRowBytes);                // [4 warps][16 rows][D + 2]
    {
        const int r0 = lane >> 2, r1 = r0 + 8, col = (lane & 3) * 2;
        float* w0 = park + ((size_t)warp * 16 + r0) * (D + 2);
        float* w1 = park + ((size_t)warp * 16 + r1) * (D + 2);
        if (r0 < heads_here) {
            if ((lane & 3) == 0) { w0[0] = m0 == -INFINITY ? -INFINITY : m0 * scale_log2; w0[1] = l0; }
#pragma unroll
            for (int i = 0; i < D / 8; ++i) *reinterpret_cast<float2*>(w0 + 2 + i * 8 + col) = make_float2(o[i][0], o[i][1]);
        }
        if (r1 < heads_here) {
            if ((lane & 3) == 0) { w1[0] = m1 == -INFINITY ? -INFINITY : m1 * scale_log2; w1[1] = l1; }
#pragma unroll
            for (int i = 0; i < D / 8; ++i) *reinterpret_cast<float2*>(w1 + 2 + i * 8 + col) = make_float2(o[i][2], o[i][3]);
        }
    }
    __syncthreads();
    // element e = (head, i) of the four warps' results folded into one (m, l, O) per head
    auto folded = [&](int e) {
        const int h = e / (D + 2), i = e % (D + 2);
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, park[((size_t)w * 16 + h) * (D + 2)]);
        if (i == 0) return M;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = park[((size_t)w * 16 + h) * (D + 2)];
            const float f = mw == -INFINITY ? 0.0f : exp2f(mw - M);
            v = fmaf(park[((size_t)w * 16 + h) * (D + 2) + i], f, v);
        }
        return v;
    };
    const int elems = heads_here * (D + 2);
    float* gathered = park + 4 * 16 * (D + 2);       // behind the parked rows: what this block merges
    __nv_bfloat16* out_row = out + (size_t)row * out_stride + (size_t)head0 * D;
    if (split == 1) {
        for (int e = tid; e < elems; e += 128) gathered[e] = folded(e);
        __syncthreads();
        for (int e = tid; e < heads_here * D; e += 128) {
            const int h = e / D, i = e % D;
            out_row[(size_t)h * D + i] = __float2bfloat16_rn(gathered[h * (D + 2) + 2 + i] * (1.0f / gathered[h * (D + 2) + 1]));
        }
        return;
    }
    if constexpr (kByLength) {
        __shared__ int counted_last;
        const int chunks = gridDim.z;
        float* mine = partial + (((size_t)row * nq + head0) * chunks + rank) * (D + 2);
        for (int e = tid; e < elems; e += 128) {
            const int h = e / (D + 2), i = e % (D + 2);
            __stcg(mine + (size_t)h * chunks * (D + 2) + i, folded(e));
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int* counter = counters + (size_t)row * gridDim.x + head_tile;
            const int before = atomicAdd(counter, 1);
            counted_last = before == split - 1;
            if (counted_last) *counter = 0;              // every block of the row has counted: ready for the next launch
        }
        __syncthreads();
        if (!counted_last) return;
        __threadfence();
        for (int h = 0; h < heads_here; ++h)
            merge_runs<kMaxRunsByLength, D, true>(partial + ((size_t)row * nq + head0 + h) * chunks * (D + 2), split,
                                                  out_row + (size_t)h * D, tid);
        return;
    }
    // Head h is merged by block h % split.  Every block sends its (m, l, O) of a head into that block's shared
    // memory, to [h / split][sender]: once all blocks are past their tiles (the barrier they arrived at
    // above), the space behind a block's parked rows is free.  After one more barrier a block finds all
    // runs of its heads in its own memory, merges them in rank order and leaves; nobody reads its memory after
    // that barrier, so none is needed at the end.
    cluster_wait();
    const uint32_t gathered_addr = s_q + 16 * kRowBytes + 4 * 16 * (D + 2) * 4;
    for (int e = tid; e < elems; e += 128) {
        const int h = e / (D + 2), i = e % (D + 2);
        st_cluster_f32(gathered_addr + (uint32_t)((((h / split) * split + rank) * (D + 2)) + i) * 4u, (uint32_t)(h % split), folded(e));
    }
    cluster_arrive();
    cluster_wait();
    if (split <= 2) merge_gathered_heads<2, D>(gathered, out_row, rank, split, heads_here, tid);
    else if (split <= 4) merge_gathered_heads<4, D>(gathered, out_row, rank, split, heads_here, tid);
    else if (split <= 8) merge_gathered_heads<8, D>(gathered, out_row, rank, split, heads_here, tid);
    else merge_gathered_heads<kMaxClusterBlocks, D>(gathered, out_row, rank, split, heads_here, tid);
}

static int g_forced_split = 0;     // > 0: blocks per (sequence, head group), for tuning

static int g_per_warp = 1;         // 0: never the kernel whose warps walk runs of their own
static int g_run_scale_q8 = 160;   // by-length kernel: a run's length in 1/256 of the mean length of the step's rows
static int g_by_length = 1;        // 0: never deal a row's pages out by length

template <int D, int kStagesKV, bool kByLength = false, bool kPerWarp = false>
static int launch_tc_stages(const void* q, int q_stride, const void* k_pool, const void* v_pool, const int32_t* page_table,
                     int page_table_stride, const int32_t* row_slot, const int32_t* row_pos, void* out, int out_stride,
                     int rows, int nq, int nkv, int window, float scale, int split, cudaStream_t stream,
                     float* partial = nullptr, int* counters = nullptr) {
    constexpr int tiles = (16 + 2 * kStagesKV * 64) * (D * 2 + 16);
    // the query rows, the four warps' parked rows, and behind them what the cluster's blocks send (at most 31 runs)
    constexpr int park = 16 * (D * 2 + 16) + (4 * 16 + 32) * (D + 2) * 4;
    constexpr int smem = tiles > park ? tiles : park;
    auto kernel = attention_decode_tc_kernel<D, kStagesKV, kByLength, kPerWarp>;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int group = nq / nkv;
    const int kv_tiles = nkv * ((group + 15) / 16);
    if (split > 8) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
    }
    const dim3 grid = kByLength ? dim3(kv_tiles, rows, split) : dim3(split, kv_tiles, rows);
    launch_kernel_clustered(kernel, grid, 128, smem, kByLength ? 1 : split, stream, (const __nv_bfloat16*)q, q_stride,
                            (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, page_table, page_table_stride,
                            row_slot, row_pos, (__nv_bfloat16*)out, out_stride, nq, nkv, window,
                            scale * 1.4426950408889634f, partial, counters, g_run_scale_q8);
    return CITLALI_LAUNCH_CHECK();
}

// Blocks per (sequence, head group) = cluster size, and key/value tiles in flight per block.  Measured at
// head size 128, 8 key/value heads, 4,096 cached tokens: one sequence 8 blocks, eight sequences 4, sixty-four
// sequences 1 (no merging at all once the grid fills the GPU twice over).  The choice depends on the batch
// alone, never on the sequences' lengths, so a captured launch stays valid.
template <int D>
static int launch_tc(const void* q, int q_stride, const void* k_pool, const void* v_pool, const int32_t* page_table,
                     int page_table_stride, const int32_t* row_slot, const int32_t* row_pos, void* out, int out_stride,
                     int rows, int nq, int nkv, int window, float scale, cudaStream_t stream,
                     float* partial, size_t partial_floats, int* counters, size_t counter_ints) {
    const int group = nq / nkv;
    const long pairs = (long)rows * nkv * ((group + 15) / 16);
    int split = 1;
    for (int s = 8; s >= 2; s /= 2)
        if (pairs * s <= 300) { split = s; break; }
    // One or few sequences in a cache laid out for more than 2,048 tokens a sequence: a cluster of sixteen (not
    // portable) a head group.  Measured at batch 1, sixteen against eight blocks: 5.3 against 5.1 us at 1,000 cached
    // tokens, 6.7 against 7.1 at 2,000, 8.3 against 9.6 at 4,000, 12.7 against 15.9 at 8,000, 25 against 31 at
    // 16,000; the table's width, unlike the lengths, is fixed for a session.
    if (pairs * 16 <= 128 && page_table_stride > 32) split = 16;
    if (g_forced_split > 0) split = g_forced_split > kMaxClusterBlocks ? kMaxClusterBlocks : g_forced_split;
    // Many rows (one block each would fill the GPU): the rows' lengths decide, on the device, which of them get
    // more than one block.  Needs the scratch for their partial results and the zeroed counters.
    if (split == 1 && g_by_length && partial != nullptr && counters != nullptr && (size_t)pairs <= counter_ints) {
        int runs = page_table_stride / kMinRunTiles;
        if (runs > kMaxRunsByLength) runs = kMaxRunsByLength;
        while (runs > 1 && (size_t)rows * nq * runs * (D + 2) > partial_floats) --runs;
        if (runs > 1)
            return launch_tc_stages<D, kKvStages, true>(q, q_stride, k_pool, v_pool, page_table, page_table_stride, row_slot,
                                                        row_pos, out, out_stride, rows, nq, nkv, window, scale, runs, stream,
                                                        partial, counters);
    }
    // One or two rows (at most a block an SM): every warp walks a run of 16-key units of its own, three units in flight
    // a warp.  Measured against the block-wide walk at batch 1: 8.1 against 8.5 us at 4,000 cached tokens, 11.5 against
    // 13.5 at 8,000, 18.0 against 23.4 at 16,000 (batch 2: 10.8 / 12.5, 17.3 / 21.6, 30.3 / 39.7); with more rows, where
    // the launch is bound by bandwidth, it gains nothing (batch 8 at 4,000: 23.9 either way).  A ring of six units a
    // warp (one block an SM) lost 3.5 us at every length: the next launch's blocks no longer fit beside this one's.
    if constexpr (D <= 128) {
        if (g_per_warp && pairs * split <= device_sm_count())
            return launch_tc_stages<D, kKvStages, false, true>(q, q_stride, k_pool, v_pool, page_table, page_table_stride, row_slot, row_pos, out,
                                                       out_stride, rows, nq, nkv, window, scale, split, stream);
        if (pairs * split <= 80)          // more blocks than that, each filling an SM, no longer fit cluster by cluster
            return launch_tc_stages<D, 6>(q, q_stride, k_pool, v_pool, page_table, page_table_stride, row_slot, row_pos, out,
                                          out_stride, rows, nq, nkv, window, scale, split, stream);
    }
    return launch_tc_stages<D, kKvStages>(q, q_stride, k_pool, v_pool, page_table, page_table_stride, row_slot, row_pos, out,
                                          out_stride, rows, nq, nkv, window, scale, split, stream);
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
    launch_kernel(attention_decode_partial_kernel<EPL, GT>, grid, kDecodeWarps * 32, smem, stream, 
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

// > 0: the tensor-core kernel uses this many blocks per (sequence, head group) (1, 2, 4, 8 or 16); 0: its own choice.
extern "C" void citlali_attention_decode_set_split(int split) { g_forced_split = split; }

// Tuning of the kernel that deals a long row's pages out by length (steps of many rows): on/off, and a run's
// length in 1/256 of the mean length of the step's rows (256: the mean itself; 0 leaves it as it is).
// Tuning: 0 turns off the form for one or few rows in which every warp walks a run of 16-key units of its own.
extern "C" void citlali_attention_decode_set_per_warp(int on) { g_per_warp = on; }

extern "C" void citlali_attention_decode_set_by_length(int on, int run_scale_q8) {
    g_by_length = on;
    if (run_scale_q8 > 0) g_run_scale_q8 = run_scale_q8;
}

// Scratch for the partials of `rows` single-token rows whose positions stay below
// `max_positions`: floats.
extern "C" size_t citlali_attention_decode_scratch_floats(int rows, int nq, int head_dim, int page_size, int max_positions) {
    const int chunk_keys = 2 * page_size;                     // the smallest chunk any kernel here uses
    const int max_chunks = (max_positions + chunk_keys - 1) / chunk_keys;
    return (size_t)rows * nq * max_chunks * (head_dim + 2);
}

// Attention of `rows` single new tokens (bfloat16).  q rows are `q_stride` elements apart;
// positions and slots are read on the device; `max_positions` bounds the positions and fixes
// the grid.  `partial` holds citlali_attention_decode_scratch_floats(...) floats.  `counters`: `counter_ints`
// 32-bit words (one per row and key/value head is enough) that are ZERO before the first call and that every call
// leaves zero; calls that share them must not overlap on the device.  Without them (nullptr) long rows of a
// large step are not dealt out by length.
extern "C" int citlali_attention_decode(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                                        const int32_t* page_table, int page_table_stride,
                                        const int32_t* row_slot, const int32_t* row_pos,
                                        void* out, int out_stride, float* partial, size_t partial_floats,
                                        int32_t* counters, size_t counter_ints,
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
    const int group = nq / nkv;
    bool tensor_cores = page_size == 64 && q_stride % 8 == 0 && (((uintptr_t)q) & 15u) == 0;
    switch (head_dim) {
        case 16: case 32: case 48: case 64: case 80: case 96: case 112: case 128: case 256: break;
        default: tensor_cores = false;
    }
    if (tensor_cores) {
        // pages of 64 and a head size the tensor-core kernel has: in steps of few rows its blocks merge their
        // partial results through distributed shared memory and the scratch is not used
#define CITLALI_TC(DD) case DD: return launch_tc<DD>(q, q_stride, k_pool, v_pool, page_table, page_table_stride, row_slot, row_pos, \
                                                      out, out_stride, rows, nq, nkv, window, scale, stream, partial, \
                                                      partial_floats, counters, counter_ints)
        switch (head_dim) {
            CITLALI_TC(16); CITLALI_TC(32); CITLALI_TC(48); CITLALI_TC(64); CITLALI_TC(80); CITLALI_TC(96); CITLALI_TC(112);
            CITLALI_TC(128); CITLALI_TC(256);
            default: break;
        }
#undef CITLALI_TC
    }
    // other head sizes and page sizes: the CUDA-core kernel writes one partial per chunk of four pages to
    // the scratch, and a second kernel merges them
    const int chunk_keys = kChunkPages * page_size;
    const int max_chunks = (max_positions + chunk_keys - 1) / chunk_keys;
    const size_t need = (size_t)rows * nq * max_chunks * (head_dim + 2);
    if ((size_t)(max_chunks + 1) * sizeof(float) > 48 * 1024) {
        // the merge kernel keeps one weight per chunk in shared memory
        set_last_error("attention_decode: %d positions in pages of %d are %d chunks, more than the merge kernel's %d",
                       max_positions, page_size, max_chunks, 48 * 1024 / 4 - 1);
        return kTooLarge;
    }
    if (partial == nullptr || partial_floats < need) {
        set_last_error("attention_decode: %zu floats of scratch are needed, %zu were given", need, partial_floats);
        return kTooLarge;
    }
    int rc = -1000;
    {
        const int gt = group <= 1 ? 1 : group <= 2 ? 2 : group <= 4 ? 4 : 8;
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
    }
    if (rc) return rc;
    dim3 grid(nq, rows);
    launch_kernel(attention_decode_combine_kernel, grid, 128, (size_t)(max_chunks + 1) * sizeof(float), stream, partial, max_chunks, row_pos, (__nv_bfloat16*)out, out_stride,
                                                              nq, head_dim, chunk_keys, window);
    return CITLALI_LAUNCH_CHECK();
}
