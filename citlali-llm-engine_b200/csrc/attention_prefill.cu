// Causal attention of whole prompts (and of any run of new tokens) over the paged cache, in
// bfloat16 on the tensor cores, without ever writing the score matrix.
//
// A block takes 64 consecutive new tokens of one sequence and one query head; each of its four
// warps owns 16 of them.  It walks the visible keys one cache page (64 keys) at a time: the
// page's keys and values are copied to shared memory with cp.async, double-buffered; scores
// S = Q K^T come from mma.sync m16n8k16 into float registers; the running maximum, the
// exponentials and the running sum are float (online softmax: when the maximum grows, sum and
// output are rescaled); P is rounded to bfloat16 and multiplied with V by the same MMA into
// float accumulators; the division by the sum happens once at the end.
//
// The formulas are the reference's (attention_scores_kernel / attention_values_kernel,
// src/compute/cuda/kernels.cu:545-649): s = q.k / sqrt(d), keys lo..p for the token at position
// p, query head j reads key/value head j / (heads / kv_heads).  The reference holds all scores
// in memory and divides per term; this kernel's order differs from it by rounding only.
//
// The new tokens' keys and values are already in the cache when this runs, so prompts, and
// runs of tokens that continue a sequence, are the same case: row r of sequence b sits at
// position past[b] + r.
#include "api.h"
#include "common.cuh"
#include "mma_common.cuh"

namespace citlali {
namespace fa {

constexpr int kTileQ = 64, kTileK = 64, kWarps = 4;

// D: head size, a multiple of 16.  Rows in shared memory are D * 2 + 16 bytes apart, which
// spreads the eight rows of an ldmatrix over all banks.
template <int D>
__global__ void __launch_bounds__(kWarps * 32)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                         const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                         const int32_t* __restrict__ page_table, int page_table_stride,
                         const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot,
                         const int32_t* __restrict__ seq_past,
                         __nv_bfloat16* __restrict__ out, int out_stride,
                         int nq, int nkv, int window, float scale_log2) {
    constexpr int kRowBytes = D * 2 + 16;
    constexpr int kTileBytes = kTileK * kRowBytes;
    constexpr int kChunksPerRow = D / 8;                     // 16-byte pieces of a row
    extern __shared__ __align__(16) uint8_t smem[];
    // [Q tile][K 0][K 1][V 0][V 1]
    const uint32_t s_q = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t s_k = s_q + kTileBytes, s_v = s_k + 2 * kTileBytes;

    dependents_may_launch();
    wait_for_predecessor();
    // blocks are handed out x fastest: all heads of the last query tile (it sees the most keys) first
    const int seq = blockIdx.z, head = blockIdx.x;
    const int row0 = seq_start[seq], n_new = seq_start[seq + 1] - row0;
    const int q0 = (gridDim.y - 1 - blockIdx.y) * kTileQ;
    if (q0 >= n_new) return;
    const int past = seq_past[seq];
    const int g = head / (nq / nkv);
    const int32_t* pages = page_table + (size_t)seq_slot[seq] * page_table_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tid = threadIdx.x;

    // the query tile: rows past the sequence's end are zeros
    for (int c = tid; c < kTileQ * kChunksPerRow; c += kWarps * 32) {
        const int r = c / kChunksPerRow, ch = c % kChunksPerRow;
        const uint32_t dst = s_q + r * kRowBytes + ch * 16;
        if (q0 + r < n_new) cp_async16(dst, q + (size_t)(row0 + q0 + r) * q_stride + (size_t)head * D + ch * 8);
        else *reinterpret_cast<uint4*>(smem + r * kRowBytes + ch * 16) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();

    // key tiles this block visits: from the first key its first row may see to the last key its last row sees
    const int last_pos = past + min(q0 + kTileQ, n_new) - 1;
    const int first_pos = past + q0;
    const int lo_key = window > 0 ? max(0, first_pos - window + 1) : 0;
    const int tile_lo = lo_key / kTileK, tile_hi = last_pos / kTileK;

    auto load_tile = [&](int tile, int buf) {
        const size_t base = ((size_t)pages[tile] * nkv + g) * kTileK * D;
        for (int c = tid; c < kTileK * kChunksPerRow; c += kWarps * 32) {
            const int r = c / kChunksPerRow, ch = c % kChunksPerRow;
            const size_t src = base + (size_t)r * D + ch * 8;
            cp_async16(s_k + buf * kTileBytes + r * kRowBytes + ch * 16, k_pool + src);
            cp_async16(s_v + buf * kTileBytes + r * kRowBytes + ch * 16, v_pool + src);
        }
    };
    load_tile(tile_lo, 0);
    cp_async_commit();

    // Q fragments of this warp's 16 rows, for every 16-wide slice of the head
    uint32_t qf[D / 16][4];
    cp_async_wait<1>();
    __syncthreads();
    {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int cbyte = (lane >> 4) * 16;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
            ldmatrix_x4(s_q + r * kRowBytes + ks * 32 + cbyte, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;      // rows lane/4 and lane/4 + 8
    const int pos0 = past + q0 + warp * 16 + (lane >> 2), pos1 = pos0 + 8;
    const int lo0 = window > 0 ? pos0 - window + 1 : 0, lo1 = window > 0 ? pos1 - window + 1 : 0;

    for (int tile = tile_lo; tile <= tile_hi; ++tile) {
        const int buf = (tile - tile_lo) & 1;
        if (tile + 1 <= tile_hi) load_tile(tile + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const uint32_t kb = s_k + buf * kTileBytes, vb = s_v + buf * kTileBytes;
        float s[kTileK / 8][4];
#pragma unroll
        for (int i = 0; i < kTileK / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
        // S = Q K^T: B fragments come from K rows (key = n, head element = k), two key groups of 8 at a time
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < kTileK / 16; ++np) {
                const int r = np * 16 + (lane & 7) + (lane >> 4) * 8;
                const int cbyte = ((lane >> 3) & 1) * 16;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(kb + r * kRowBytes + ks * 32 + cbyte, b0, b1, b2, b3);
                mma_16816(s[2 * np], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                mma_16816(s[2 * np + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
            }
        }
        // mask, then the running maximum of each row (shared by the four lanes of a row)
        const int key_base = tile * kTileK + (lane & 3) * 2;
        float mx0 = -INFINITY, mx1 = -INFINITY;
        // only tiles that reach past the warp's first row, or start before its last row's window, need the mask
        const int warp_pos = past + q0 + warp * 16;
        const bool masked = tile * kTileK + kTileK - 1 > warp_pos || (window > 0 && tile * kTileK < warp_pos + 15 - window + 1);
        if (masked) {
#pragma unroll
            for (int i = 0; i < kTileK / 8; ++i) {
                const int key = key_base + i * 8;
                if (key > pos0 || key < lo0) s[i][0] = -INFINITY;
                if (key + 1 > pos0 || key + 1 < lo0) s[i][1] = -INFINITY;
                if (key > pos1 || key < lo1) s[i][2] = -INFINITY;
                if (key + 1 > pos1 || key + 1 < lo1) s[i][3] = -INFINITY;
            }
        }
#pragma unroll
        for (int i = 0; i < kTileK / 8; ++i) {
            mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
            mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // a row that has seen no key yet keeps maximum -inf; use 0 in its exponents so nothing is NaN
        const float ref0 = mn0 == -INFINITY ? 0.0f : mn0 * scale_log2, ref1 = mn1 == -INFINITY ? 0.0f : mn1 * scale_log2;
        const float a0 = fast_exp2(m0 * scale_log2 - ref0), a1 = fast_exp2(m1 * scale_log2 - ref1);
        m0 = mn0; m1 = mn1;
        float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
        for (int i = 0; i < kTileK / 8; ++i) {
            s[i][0] = fast_exp2(s[i][0] * scale_log2 - ref0); s[i][1] = fast_exp2(s[i][1] * scale_log2 - ref0);
            s[i][2] = fast_exp2(s[i][2] * scale_log2 - ref1); s[i][3] = fast_exp2(s[i][3] * scale_log2 - ref1);
            sum0 += s[i][0] + s[i][1];
            sum1 += s[i][2] + s[i][3];
        }
        l0 = l0 * a0 + sum0; l1 = l1 * a1 + sum1;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
        // O += P V: P's accumulator layout is the A-fragment layout; V's B fragments need the transpose load
#pragma unroll
        for (int kk = 0; kk < kTileK / 16; ++kk) {
            const uint32_t p0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), p1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            const uint32_t p2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), p3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < D / 16; ++np) {
                const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int cbyte = np * 32 + (lane >> 4) * 16;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(vb + r * kRowBytes + cbyte, b0, b1, b2, b3);
                mma_16816(o[2 * np], p0, p1, p2, p3, b0, b1);
                mma_16816(o[2 * np + 1], p0, p1, p2, p3, b2, b3);
            }
        }
        __syncthreads();          // everyone is done with this buffer before the next load overwrites it
    }
    cp_async_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, inv1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
    const int r0 = q0 + warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        if (r0 < n_new)
            *reinterpret_cast<uint32_t*>(out + (size_t)(row0 + r0) * out_stride + (size_t)head * D + i * 8 + col) =
                pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
        if (r1 < n_new)
            *reinterpret_cast<uint32_t*>(out + (size_t)(row0 + r1) * out_stride + (size_t)head * D + i * 8 + col) =
                pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
}

template <int D>
static int launch(const void* q, int q_stride, const void* k_pool, const void* v_pool, const int32_t* page_table,
                  int page_table_stride, const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_past,
                  void* out, int out_stride, int sequences, int max_new, int nq, int nkv, int window, float scale,
                  cudaStream_t stream) {
    constexpr int smem = 5 * kTileK * (D * 2 + 16);
    auto kernel = attention_prefill_kernel<D>;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(nq, (max_new + kTileQ - 1) / kTileQ, sequences);
    launch_kernel(kernel, grid, kWarps * 32, smem, stream, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_pool,
                                                 (const __nv_bfloat16*)v_pool, page_table, page_table_stride, seq_start,
                                                 seq_slot, seq_past, (__nv_bfloat16*)out, out_stride, nq, nkv, window,
                                                 scale * 1.4426950408889634f);
    return CITLALI_LAUNCH_CHECK();
}

}  // namespace fa
}  // namespace citlali

using namespace citlali;

// 1 if citlali_attention_prefill has a kernel for this head size and page size.
extern "C" int citlali_attention_prefill_supports(int head_dim, int page_size) {
    if (page_size != fa::kTileK) return 0;
    switch (head_dim) {
        case 16: case 32: case 48: case 64: case 80: case 96: case 112: case 128: case 256: return 1;
        default: return 0;
    }
}

// Attention of the new tokens of `sequences` sequences (bfloat16, pages of 64).  Sequence b owns
// rows seq_start[b] .. seq_start[b+1]-1, at positions seq_past[b] + i of slot seq_slot[b];
// `max_new` is the largest number of new tokens of any sequence.  The 64-bit row pitch of q
// (q_stride elements) and of out must keep rows 16-byte aligned.
extern "C" int citlali_attention_prefill(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                                         const int32_t* page_table, int page_table_stride,
                                         const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_past,
                                         void* out, int out_stride, int sequences, int max_new,
                                         int nq, int nkv, int head_dim, int page_size, int window, float scale,
                                         cudaStream_t stream) {
    if (sequences <= 0 || max_new <= 0) return 0;
    if (!citlali_attention_prefill_supports(head_dim, page_size)) {
        set_last_error("attention_prefill: no kernel for head size %d with pages of %d (head sizes 16..128 in steps of 16 "
                       "and 256, pages of 64)", head_dim, page_size);
        return kBadShape;
    }
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || max_new / fa::kTileQ >= 65535 || sequences > 65535) {
        set_last_error("attention_prefill: bad head counts (%d over %d) or too many sequences (%d)", nq, nkv, sequences);
        return kBadShape;
    }
    if (q_stride % 8 != 0 || out_stride % 2 != 0 || ((uintptr_t)q & 15u) || ((uintptr_t)out & 3u)) {
        set_last_error("attention_prefill: query rows must be 16-byte aligned (row pitch %d elements)", q_stride);
        return kBadAlignment;
    }
#define CITLALI_FA(DD) case DD: return fa::launch<DD>(q, q_stride, k_pool, v_pool, page_table, page_table_stride, seq_start, \
                                                      seq_slot, seq_past, out, out_stride, sequences, max_new, nq, nkv, window, scale, stream)
    switch (head_dim) {
        CITLALI_FA(16); CITLALI_FA(32); CITLALI_FA(48); CITLALI_FA(64); CITLALI_FA(80); CITLALI_FA(96); CITLALI_FA(112);
        CITLALI_FA(128); CITLALI_FA(256);
    }
#undef CITLALI_FA
    return kBadShape;
}
