// Causal attention of runs of new tokens over the paged cache on the fifth-generation tensor
// cores, for head size 128 and pages of 64 keys.
//
// A block takes 128 consecutive new tokens of one sequence and one query head and walks the
// visible keys 128 at a time (two cache pages).  Three roles run concurrently:
//   warp 4, one lane: TMA producer.  The query tile once, then a key tile and a value tile at a
//                     time (128-byte swizzle; a tile is two 64-wide halves of the head); the next
//                     key tile is fetched as soon as the scores of the current one are computed.
//   warp 5, one lane: MMA issuer.  S = Q K^T (tcgen05.mma, both operands K-major in shared
//                     memory) into tensor memory; O += P V with P read from tensor memory (it
//                     overwrites the first half of S) and V, as stored (head dimension
//                     contiguous), as an MN-major shared-memory operand.
// A block needs 97 KB of shared memory and 256 columns of tensor memory, so two blocks share an SM:
// while one block's softmax warps work, the other block's MMAs run.
//   warps 0-3:        softmax.  Each thread owns one query row: it reads its 128 scores from
//                     tensor memory, keeps the running reference maximum and sum in float
//                     (no shuffles), writes P as bfloat16 back to tensor memory, and rescales
//                     its row of O only when the maximum has grown by more than 2^8 (the sum
//                     uses the same reference, so the result is exact).  At the end it divides
//                     its row of O by the sum and stores it.
//
// Formulas: the reference's (attention_scores_kernel / attention_values_kernel,
// src/compute/cuda/kernels.cu:545-649): s = q.k / sqrt(d), keys lo..p for the token at position
// p, query head j reads key/value head j / (heads / kv_heads); softmax and sums in float.
// Every mbarrier wait is bounded and reports through the error word.
#include "api.h"
#include "common.cuh"
#include "tc_common.cuh"

namespace citlali {
namespace fatc {

using namespace tc;

constexpr int kD = 128, kTileQ = 128, kTileK = 128, kPage = 64;
constexpr int kThreads = 192;
constexpr uint32_t kHalfTile = 128 * 128;              // bytes of [128 rows x 64 bfloat16]
constexpr uint32_t kTileBytes = 2 * kHalfTile;         // [128 x 128] bfloat16
// tensor memory columns
constexpr uint32_t kColS = 0, kColP = 0, kColO = 128, kTmemCols = 256;     // P overwrites the scores it came from

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
// 32 consecutive columns of this thread's lane into r[0..31] (no wait).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] . B[smem]: A is P, 16 bfloat16 per row in 8 columns.
__device__ __forceinline__ void mma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

// Shared-memory descriptor of an MN-major operand with 128-byte swizzle: rows of 128 bytes hold 64
// consecutive elements of the MN dimension, consecutive rows are consecutive K indices, groups of 8
// rows are 1024 bytes apart, and the next 64 MN elements start `mn_step` bytes further.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t mn_step) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFFu);
    d |= (uint64_t)((mn_step >> 4) & 0x3FFFu) << 16;     // leading byte offset: along MN
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset: along K
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct Params {
    const int32_t* page_table; int page_table_stride;
    const int32_t* seq_start; const int32_t* seq_slot; const int32_t* seq_past;
    __nv_bfloat16* out; int out_stride;
    int nq, nkv, window;
    float scale_log2;
    int32_t* error_flag;
};

__global__ void __launch_bounds__(kThreads, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, Params p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t q_bar, k_full, v_full, k_empty, v_empty, s_full, p_full, o_done;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;

    dependents_may_launch();
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t s_q = base, s_k = base + kTileBytes, s_v = s_k + kTileBytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        abort_word = 0;
        mbar_init(smem_u32(&q_bar), 1);
        mbar_init(smem_u32(&k_full), 1); mbar_init(smem_u32(&v_full), 1);
        mbar_init(smem_u32(&k_empty), 1); mbar_init(smem_u32(&v_empty), 1);
        mbar_init(smem_u32(&s_full), 1);
        mbar_init(smem_u32(&p_full), 4);
        mbar_init(smem_u32(&o_done), 1);
        fence_barrier_init();
        fence_async_proxy();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    wait_for_predecessor();                                  // everything below reads what earlier kernels wrote
    // blocks are handed out x fastest: all heads of the last query tile (the one that sees the most
    // keys) first, then all heads of the tile before it, and so on
    const int seq = blockIdx.z, head = blockIdx.x;
    const int row0 = p.seq_start[seq], n_new = p.seq_start[seq + 1] - row0;
    const int q0 = (gridDim.y - 1 - blockIdx.y) * kTileQ;
    const bool active = q0 < n_new;
    const int past = p.seq_past[seq];
    const int g = head / (p.nq / p.nkv);
    const int32_t* pages = p.page_table + (size_t)p.seq_slot[seq] * p.page_table_stride;
    const int first_pos = past + q0, last_pos = past + min(q0 + kTileQ, n_new) - 1;
    const int lo_key = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
    const int tile_lo = lo_key / kTileK, tile_hi = last_pos / kTileK;
    const int tiles = active ? tile_hi - tile_lo + 1 : 0;

    if (warp == 4) {
        if (lane == 0 && active) {
            mbar_arrive_expect_tx(smem_u32(&q_bar), kTileBytes);
            tma_load_2d(s_q, &map_q, head * kD, row0 + q0, smem_u32(&q_bar));
            tma_load_2d(s_q + kHalfTile, &map_q, head * kD + 64, row0 + q0, smem_u32(&q_bar));
            for (int t = 0; t < tiles; ++t) {
                const int key0 = (tile_lo + t) * kTileK;
                // two pages per tile; a page that lies wholly past the last visible key is not fetched (the
                // first page stands in): its scores are masked and its values are multiplied by zeros
                const int page_a = pages[key0 / kPage];
                const bool second = key0 + kPage <= last_pos;
                const int page_b = second ? pages[key0 / kPage + 1] : page_a;
                const int ra = (page_a * p.nkv + g) * kPage, rb = (page_b * p.nkv + g) * kPage;
                const uint32_t kb = smem_u32(&k_full), vb = smem_u32(&v_full);
                if (!mbar_wait(smem_u32(&k_empty), (t & 1u) ^ 1u, abort_flag, p.error_flag, 201)) break;
                mbar_arrive_expect_tx(kb, kTileBytes);
                tma_load_2d(s_k, &map_k, 0, ra, kb);
                tma_load_2d(s_k + 64 * 128, &map_k, 0, rb, kb);
                tma_load_2d(s_k + kHalfTile, &map_k, 64, ra, kb);
                tma_load_2d(s_k + kHalfTile + 64 * 128, &map_k, 64, rb, kb);
                if (!mbar_wait(smem_u32(&v_empty), (t & 1u) ^ 1u, abort_flag, p.error_flag, 210)) break;
                mbar_arrive_expect_tx(vb, kTileBytes);
                tma_load_2d(s_v, &map_v, 0, ra, vb);
                tma_load_2d(s_v + 64 * 128, &map_v, 0, rb, vb);
                tma_load_2d(s_v + kHalfTile, &map_v, 64, ra, vb);
                tma_load_2d(s_v + kHalfTile + 64 * 128, &map_v, 64, rb, vb);
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        if (lane == 0 && active) {
            constexpr uint32_t idesc_qk = instr_desc_bf16(kTileQ, kTileK);
            constexpr uint32_t idesc_pv = instr_desc_bf16(kTileQ, kD) | (1u << 16);        // B is MN-major
            // MMAs of one thread run in the order they are issued, so the scores of tile t+1, issued after
            // P V of tile t, overwrite P only when that product has read it
            auto issue_qk = [&]() {
#pragma unroll
                for (int ks = 0; ks < kD / 16; ++ks) {
                    const uint32_t half = (ks >> 2) * kHalfTile, off = (ks & 3) * 32;
                    mma_bf16(tmem + kColS, smem_desc_sw128(s_q + half, off), smem_desc_sw128(s_k + half, off),
                             idesc_qk, ks > 0 ? 1u : 0u);
                }
                mma_commit(smem_u32(&k_empty));
                mma_commit(smem_u32(&s_full));
            };
            bool ok = mbar_wait(smem_u32(&q_bar), 0, abort_flag, p.error_flag, 202);
            if (ok) ok = mbar_wait(smem_u32(&k_full), 0, abort_flag, p.error_flag, 203);
            if (ok) { tc_fence_after(); issue_qk(); }
            for (int t = 0; t < tiles && ok; ++t) {
                if (!mbar_wait(smem_u32(&p_full), t & 1u, abort_flag, p.error_flag, 205)) { ok = false; break; }
                if (!mbar_wait(smem_u32(&v_full), t & 1u, abort_flag, p.error_flag, 206)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int j = 0; j < kTileK / 16; ++j)
                    mma_bf16_ts(tmem + kColO, tmem + kColP + j * 8, smem_desc_mn_sw128(s_v + j * 16 * 128, kHalfTile), idesc_pv,
                                (t > 0 || j > 0) ? 1u : 0u);
                mma_commit(smem_u32(&v_empty));
                mma_commit(smem_u32(&o_done));
                if (t + 1 < tiles) {
                    if (!mbar_wait(smem_u32(&k_full), (t + 1) & 1u, abort_flag, p.error_flag, 204)) { ok = false; break; }
                    tc_fence_after();
                    issue_qk();
                }
            }
        }
        __syncwarp();
    } else if (active) {
        // softmax: this thread owns query row `r`
        const int r = warp * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        const int pos = past + q0 + r;
        const int lo = p.window > 0 ? pos - p.window + 1 : 0;
        float m_ref = -INFINITY, l = 0.0f;                    // reference maximum (raw score units) and sum
        bool ok = true;
        for (int t = 0; t < tiles && ok; ++t) {
            const int key0 = (tile_lo + t) * kTileK;
            const uint32_t s_addr = tmem + lane_addr + kColS;
            if (!mbar_wait(smem_u32(&s_full), t & 1u, abort_flag, p.error_flag, 207)) { ok = false; break; }
            tc_fence_after();
            const bool masked = key0 + kTileK - 1 > past + q0 + warp * 32 || (p.window > 0 && key0 < past + q0 + warp * 32 + 31 - p.window + 1);
            // The row's 128 scores, 64 at a time to keep registers for two blocks per SM: maximum of the
            // first half (dropped), then the second half (kept), then the first half again.
            uint32_t lo_half[64], hi_half[64];
            auto load_half = [&](uint32_t* dst, int c_base) {
                tmem_ld32(s_addr + c_base, dst);
                tmem_ld32(s_addr + c_base + 32, dst + 32);
                tmem_ld_wait();
                if (masked) {
#pragma unroll
                    for (int c = 0; c < 64; ++c) {
                        const int key = key0 + c_base + c;
                        if (key > pos || key < lo) dst[c] = 0xff800000u;          // -inf
                    }
                }
            };
            float mx = -INFINITY;
            load_half(lo_half, 0);
#pragma unroll
            for (int c = 0; c < 64; ++c) mx = fmaxf(mx, __uint_as_float(lo_half[c]));
            load_half(hi_half, 64);
#pragma unroll
            for (int c = 0; c < 64; ++c) mx = fmaxf(mx, __uint_as_float(hi_half[c]));
            // grow the reference only when the maximum has run away by more than 2^8
            float alpha = 1.0f;
            const bool grow = (mx - m_ref) * p.scale_log2 > 8.0f || m_ref == -INFINITY;
            if (grow && mx > -INFINITY) {
                alpha = m_ref == -INFINITY ? 0.0f : ex2((m_ref - mx) * p.scale_log2);
                m_ref = mx;
                l *= alpha;
            }
            const bool rescale = t > 0 && __any_sync(0xffffffffu, alpha != 1.0f);
            const float ref = m_ref == -INFINITY ? 0.0f : m_ref * p.scale_log2;
            float sum = 0.0f;
            auto exp_pack = [&](uint32_t* h) {                // 64 scores -> 32 registers of two bfloat16
#pragma unroll
                for (int c = 0; c < 64; c += 2) {
                    const float a = ex2(fmaf(__uint_as_float(h[c]), p.scale_log2, -ref));
                    const float b = ex2(fmaf(__uint_as_float(h[c + 1]), p.scale_log2, -ref));
                    sum += a + b;
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(a, b);
                    h[c >> 1] = *reinterpret_cast<uint32_t*>(&h2);
                }
            };
            exp_pack(hi_half);
            load_half(lo_half, 0);
            exp_pack(lo_half);
            l += sum;
            // O must be quiet before it is rescaled (P V of the tile before has ended by then anyway: the
            // scores of this tile were issued after it)
            if (rescale) {
                if (!mbar_wait(smem_u32(&o_done), (t - 1) & 1u, abort_flag, p.error_flag, 208)) { ok = false; break; }
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < kD; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem + lane_addr + kColO + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * alpha);
                    tmem_st32(tmem + lane_addr + kColO + c0, v);
                }
            }
            tmem_st32(tmem + lane_addr + kColP, lo_half);
            tmem_st32(tmem + lane_addr + kColP + 32, hi_half);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full));
        }
        if (ok && tiles > 0 && mbar_wait(smem_u32(&o_done), (tiles - 1) & 1u, abort_flag, p.error_flag, 209)) {
            tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const bool store = q0 + r < n_new;
            __nv_bfloat16* dst = p.out + (size_t)(row0 + q0 + r) * p.out_stride + (size_t)head * kD;
#pragma unroll 1
            for (int c0 = 0; c0 < kD; c0 += 32) {
                uint32_t ov[32];
                tmem_ld32(tmem + lane_addr + kColO + c0, ov);
                tmem_ld_wait();
                if (store) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(ov[c + 2 * e]) * inv, __uint_as_float(ov[c + 2 * e + 1]) * inv);
                            w[e] = *reinterpret_cast<uint32_t*>(&h2);
                        }
                        *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return (EncodeTiledFn)f;
    }();
    return fn;
}

// [rows, row_elems] bfloat16, row pitch `pitch_elems`, as boxes of [box_rows, 64] with 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_elems, uint64_t pitch_elems, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_last_error("attention_prefill_tc: the driver does not provide cuTensorMapEncodeTiled");
        return kNoDriverEntry;
    }
    cuuint64_t dims[2] = {row_elems, rows};
    cuuint64_t strides[1] = {pitch_elems * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("attention_prefill_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
        return kBadShape;
    }
    return 0;
}

}  // namespace fatc
}  // namespace citlali

using namespace citlali;

// 1 if citlali_attention_prefill_tc takes this geometry.
extern "C" int citlali_attention_prefill_tc_supports(int head_dim, int page_size) {
    return head_dim == fatc::kD && page_size == fatc::kPage;
}

// As citlali_attention_prefill, on tcgen05, for head size 128 and pages of 64.  `total_rows` is the
// number of rows of q (all sequences), `pool_pages` the number of pages of the layer's pools.
extern "C" int citlali_attention_prefill_tc(const void* q, int q_stride, int total_rows,
                                            const void* k_pool, const void* v_pool, int pool_pages,
                                            const int32_t* page_table, int page_table_stride,
                                            const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_past,
                                            void* out, int out_stride, int sequences, int max_new,
                                            int nq, int nkv, int head_dim, int page_size, int window, float scale,
                                            int32_t* error_flag, cudaStream_t stream) {
    if (sequences <= 0 || max_new <= 0) return 0;
    if (!citlali_attention_prefill_tc_supports(head_dim, page_size)) {
        set_last_error("attention_prefill_tc: head size %d with pages of %d is not taken (128 and 64 only)", head_dim, page_size);
        return kBadShape;
    }
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || max_new / fatc::kTileQ >= 65535 || sequences > 65535) {
        set_last_error("attention_prefill_tc: bad head counts (%d over %d) or too many sequences (%d)", nq, nkv, sequences);
        return kBadShape;
    }
    if (q_stride % 8 != 0 || out_stride % 8 != 0 || ((uintptr_t)q & 15u) || ((uintptr_t)out & 15u) ||
        ((uintptr_t)k_pool & 15u) || ((uintptr_t)v_pool & 15u)) {
        set_last_error("attention_prefill_tc: rows of q and out must be 16-byte aligned");
        return kBadAlignment;
    }
    CUtensorMap mq, mk, mv;
    int rc;
    if ((rc = fatc::make_map(&mq, q, (uint64_t)total_rows, (uint64_t)nq * head_dim, (uint64_t)q_stride, fatc::kTileQ))) return rc;
    const uint64_t pool_rows = (uint64_t)pool_pages * nkv * page_size;
    if ((rc = fatc::make_map(&mk, k_pool, pool_rows, head_dim, head_dim, fatc::kPage))) return rc;
    if ((rc = fatc::make_map(&mv, v_pool, pool_rows, head_dim, head_dim, fatc::kPage))) return rc;
    fatc::Params p;
    p.page_table = page_table; p.page_table_stride = page_table_stride;
    p.seq_start = seq_start; p.seq_slot = seq_slot; p.seq_past = seq_past;
    p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
    p.nq = nq; p.nkv = nkv; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.error_flag = error_flag;
    const size_t smem = (size_t)3 * fatc::kTileBytes + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(fatc::attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(nq, (max_new + fatc::kTileQ - 1) / fatc::kTileQ, sequences);
    launch_kernel(fatc::attention_prefill_tc_kernel, grid, fatc::kThreads, smem, stream, mq, mk, mv, p);
    return CITLALI_LAUNCH_CHECK();
}
