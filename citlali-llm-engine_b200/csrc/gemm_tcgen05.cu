// y[M, N] = x[M, K] . w[N, K]^T in bfloat16 on the fifth-generation tensor cores.
//
// One persistent block per SM slot walks over work units (output tile x K split).  Inside a
// block three roles run concurrently:
//   warp 0, one lane: TMA producer.  Loads [128 x 64] and [BN x 64] bfloat16 tiles of the two
//                     operands into a ring of shared-memory stages (128-byte swizzle).
//   warp 1, one lane: MMA issuer.  Four tcgen05.mma (K = 16 each) per stage into a float
//                     accumulator in tensor memory; tcgen05.commit frees the stage, and after
//                     the last K block hands the accumulator to the epilogue.
//   warps 2-5:        epilogue.  tcgen05.ld the accumulator (each warp its 32 TMEM lanes),
//                     then store / add to the float32 residual / write a split-K partial.
// Two accumulator stages let the epilogue of one unit overlap the main loop of the next.
//
// Both operands are K-major, as the reference stores its weights (kernels.cu:387).  With many
// rows of x ("normal": prompts) the MMA's 128-row operand is x and the BN-row operand is w.
// With few rows ("swapped": decoding) the 128-row operand is w, so the weights stream through
// the wide side at full rate and the few rows of x are the narrow side; K is then split over
// several blocks so that every SM streams weights.  The splits of a tile are one thread-block
// cluster: each block sends its float32 partial sums through distributed shared memory to the
// block that owns that part of the tile, which adds them in split order and writes the result.
// The split depends on the shape alone, never on the batch, so a row's result does not depend
// on what else is in the step.
//
// Every wait on an mbarrier gives up after a time limit, raises the error word and makes the
// block leave through the normal exit (TMEM freed, copies in flight awaited).
#include "api.h"
#include "common.cuh"
#include "tc_common.cuh"
#include "tc_host.h"

#include <cstdio>
#include <map>
#include <mutex>
#include <tuple>

namespace citlali {
namespace tc {

constexpr int kBM = 128, kBK = 64, kAccStages = 2;
// two role warps and the epilogue warps: eight for prompts, where a tile's epilogue must not outlast the next
// tile's main loop, and for 64 and more rows of x with the weights as the 128-row operand (a block's only
// epilogue is not hidden by anything there); four for fewer rows
__host__ __device__ constexpr int epilogue_warps(bool swapped, int bn) { return swapped && bn < 64 ? 4 : 8; }
__host__ __device__ constexpr int threads_for(bool swapped, int bn) { return 64 + 32 * epilogue_warps(swapped, bn); }
constexpr int kMaxSplits = 8;       // a cluster's portable size
constexpr int kMaxSwappedRows = 256;

struct GemmParams {
    void* out;             // [M, N] ([M, N / 2] under the gate epilogue)
    int out_kind;
    int M, N, K;           // the product's logical shape: y[M, N] = x[M, K] w[N, K]^T
    int rows_a, rows_b;    // rows of the 128-row operand and of the BN-row operand
    int splits;            // K is cut into this many ranges of whole 64-blocks
    int32_t* error_flag;
    // Few rows of x only (the swapped form), for a layer norm that lives in the products around it instead of in a
    // kernel of its own.  A product that adds into the float32 residual rows (kAddF32) may also EMIT what the norm of the
    // updated rows needs: the rows as bfloat16 and the sums of their squares over each 32 consecutive features.  The
    // product that follows reads those rows as its x and SCALES its result rows by rsqrt(sum of squares / dim + eps)
    // (its weights carry the norm's gain): y = (x . (g * w)^T) * inv_rms(x) = (x * inv_rms(x) * g) . w^T.
    __nv_bfloat16* emit_rows;      // [M, N] or null
    float* emit_sumsq;             // [M, N / 32] (N a multiple of 32)
    const float* scale_sumsq;      // [M, scale_groups] or null: sums of squares of the rows of this product's x
    int scale_groups;
    int scale_dim;
    float scale_eps;
};

template <int BN>
constexpr int stages_for(bool swapped) {
    // Swapped (few rows of x): two blocks per SM of about 100 KB each (one of 192 KB for tiles of 256 rows of
    // x); up to 64 rows of x the split-K receive area (BN x 512 bytes) lies behind the ring, wider tiles
    // reuse the ring for it (and need a cluster barrier more).  For 64 rows that means three stages instead of
    // four; measured on the four products of a layer: 14.2 / 10.6 / 40.0 / 21.2 us against 14.5 / 12.8 / 38.9 / 22.3.
    // Normal: one block of
    // about 200 KB, and 20 KB behind the ring for the epilogue warps.
    return swapped ? (BN <= 16 ? 5 : BN <= 32 ? 4 : BN <= 128 ? 3 : 4) : (BN <= 128 ? 6 : BN <= 192 ? 5 : 4);
}

__device__ __forceinline__ void red_add_f32(float* addr, float v) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_f4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ float4 ld_shared_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

template <int BN, bool kSwapped>
__global__ void __launch_bounds__(threads_for(kSwapped, BN), (kSwapped && BN <= 128) ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmParams p) {
    constexpr int kStages = stages_for<BN>(kSwapped);
    constexpr uint32_t kBytesA = kBM * kBK * 2, kBytesB = BN * kBK * 2;
    constexpr uint32_t kTmemCols = (kAccStages * BN) <= 32 ? 32 : (kAccStages * BN) <= 64 ? 64 : (kAccStages * BN) <= 128 ? 128
                                   : (kAccStages * BN) <= 256 ? 256 : 512;        // a power of two
    constexpr uint32_t kIdesc = instr_desc_bf16(kBM, BN);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], acc_full_bar[kAccStages], acc_empty_bar[kAccStages];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_word;
    __shared__ float row_scale[kSwapped ? BN : 1];            // see GemmParams::scale_sumsq
    volatile int* abort_flag = &abort_word;
    // An emitting product with a split K: the old residual values of the one unit this warp will own, fetched while the
    // K loop runs (they have been final since the kernel ahead ended; fetched after the sums they would be a load from
    // memory at the very end of the kernel, which costs more than the norm kernel this saves)
    float x_old[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    bool have_old = false;

    dependents_may_launch();
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;            // tile storage starts on a 1024-byte boundary
    const uint32_t smem_a = tiles, smem_b = tiles + kStages * kBytesA;
    // Split K: where the other blocks of the cluster put their partial sums of this block's share of the
    // tile.  Behind the ring for narrow tiles; over the ring for wide ones, which then need a cluster
    // barrier between the last MMA of every block and the first partial sent.
    constexpr bool kRecvInRing = BN >= 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t behind_ring = tiles + kStages * (kBytesA + kBytesB);
    const uint32_t recv = kRecvInRing ? tiles : behind_ring;
    // normal form: an area for each epilogue warp to turn its values round in (tc_common.cuh)
    const uint32_t epilogue_stage = behind_ring + (uint32_t)((warp - 2) & 7) * kEpilogueStageBytes;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        abort_word = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int a = 0; a < kAccStages; ++a) { mbar_init(smem_u32(&acc_full_bar[a]), 1); mbar_init(smem_u32(&acc_empty_bar[a]), epilogue_warps(kSwapped, BN)); }
        fence_barrier_init();
        fence_async_proxy();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int tiles_a = (p.rows_a + kBM - 1) / kBM, tiles_b = (p.rows_b + BN - 1) / BN;
    const int kblocks = (p.K + kBK - 1) / kBK;
    const int kb_per_split = (kblocks + p.splits - 1) / p.splits;
    const int units = tiles_a * tiles_b * p.splits;

    // unit -> (a tile, b tile, split): the split runs fastest (the blocks of a cluster), then the tile of the
    // 128-row operand.  Normal form (no split): blocks that run together share a weight tile.
    auto decode = [&](int u, int& ta, int& tb, int& sp) {
        sp = u % p.splits; u /= p.splits; ta = u % tiles_a; tb = u / tiles_a;
    };

    if (warp == 0) {
        if (lane == 0) {
            // Visit this block's (unit, K block) pairs in order; `body` returns false to stop.
            auto for_each = [&](auto&& body) {
                uint32_t it = 0;
                for (int u = blockIdx.x; u < units; u += gridDim.x) {
                    int ta, tb, sp;
                    decode(u, ta, tb, sp);
                    const int kb0 = sp * kb_per_split, kb1 = min(kblocks, kb0 + kb_per_split);
                    for (int kb = kb0; kb < kb1; ++kb, ++it)
                        if (!body(it, ta, tb, kb)) return it;
                }
                return it;
            };
            // The weights are written by no kernel, so the first ring of weight tiles is fetched before
            // the kernel ahead of this one has finished; the rows of x only after it has.
            auto load_weights = [&](int s, int ta, int tb, int kb, uint32_t bar) {
                if (kSwapped) tma_load_2d(smem_a + s * kBytesA, &map_a, kb * kBK, ta * kBM, bar);
                else tma_load_2d(smem_b + s * kBytesB, &map_b, kb * kBK, tb * BN, bar);
            };
            auto load_rows = [&](int s, int ta, int tb, int kb, uint32_t bar) {
                if (kSwapped) tma_load_2d(smem_b + s * kBytesB, &map_b, kb * kBK, tb * BN, bar);
                else tma_load_2d(smem_a + s * kBytesA, &map_a, kb * kBK, ta * kBM, bar);
            };
            const uint32_t early = for_each([&](uint32_t it, int ta, int tb, int kb) {
                if (it >= (uint32_t)kStages) return false;
                const uint32_t bar = smem_u32(&full_bar[it]);
                mbar_arrive_expect_tx(bar, kBytesA + kBytesB);
                load_weights(it, ta, tb, kb, bar);
                return true;
            });
            wait_for_predecessor();
            bool ok = true;
            const uint32_t issued = for_each([&](uint32_t it, int ta, int tb, int kb) {
                const int s = it % kStages;
                const uint32_t bar = smem_u32(&full_bar[s]);
                if (it < early) {
                    load_rows(s, ta, tb, kb, bar);
                    return true;
                }
                if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / kStages) & 1u) ^ 1u, abort_flag, p.error_flag, 101)) { ok = false; return false; }
                mbar_arrive_expect_tx(bar, kBytesA + kBytesB);
                load_weights(s, ta, tb, kb, bar);
                load_rows(s, ta, tb, kb, bar);
                return true;
            });
            if (!ok) {
                // leaving early: let the copies this thread issued land before shared memory goes away
                const uint32_t first = issued > (uint32_t)kStages ? issued - kStages : 0u;
                for (uint32_t j = first; j < issued; ++j) {
                    const uint32_t bar = smem_u32(&full_bar[j % kStages]);
                    const uint64_t start = global_timer();
                    while (!mbar_try_wait(bar, (j / kStages) & 1u) && global_timer() - start < 100000000ull) {}
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // The tensor core takes few MMAs ahead of the one it runs, so what this thread does between the MMAs of
            // one K block and those of the next is time the tensor core stands still: the stage and its phase
            // are counted, not divided, and a stage's descriptors are the first stage's plus a constant (the
            // address field counts 16-byte units; 32 bytes on for each 16-element K slice).
            uint32_t acc_it = 0, stage = 0, phase = 0;
            const uint64_t desc_a0 = smem_desc_sw128(smem_a, 0), desc_b0 = smem_desc_sw128(smem_b, 0);
            const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
            bool ok = true;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++acc_it) {
                int ta, tb, sp;
                decode(u, ta, tb, sp);
                const int kb0 = sp * kb_per_split, kb1 = min(kblocks, kb0 + kb_per_split);
                const int as = acc_it % kAccStages;
                if (!mbar_wait(smem_u32(&acc_empty_bar[as]), ((acc_it / kAccStages) & 1u) ^ 1u, abort_flag, p.error_flag, 102)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + as * BN;
                uint32_t accumulate = 0;
                // whether the stage of the K block about to be multiplied has landed is looked up before the MMAs of
                // the block ahead of it are issued, so that between two blocks' MMAs there is only the commit
                bool landed = kb0 < kb1 && mbar_try_wait(full0 + stage * 8u, phase);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!landed && !mbar_wait(full0 + stage * 8u, phase, abort_flag, p.error_flag, 103)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t da = desc_a0 + (uint64_t)(stage * (kBytesA >> 4)), db = desc_b0 + (uint64_t)(stage * (kBytesB >> 4));
                    const uint32_t this_empty = empty0 + stage * 8u;
                    if (++stage == (uint32_t)kStages) { stage = 0; phase ^= 1u; }
                    landed = kb + 1 < kb1 && mbar_try_wait(full0 + stage * 8u, phase);
                    mma_bf16(tmem_d, da, db, kIdesc, accumulate);
                    mma_bf16(tmem_d, da + 2, db + 2, kIdesc, 1u);
                    mma_bf16(tmem_d, da + 4, db + 4, kIdesc, 1u);
                    mma_bf16(tmem_d, da + 6, db + 6, kIdesc, 1u);
                    mma_commit(this_empty);
                    accumulate = 1u;
                }
                if (ok) mma_commit(smem_u32(&acc_full_bar[as]));
            }
        }
        __syncwarp();
    } else {
        const int quarter = warp & 3;                       // the TMEM lanes this warp may read: 32 * quarter ..
        float* outf = (float*)p.out;
        __nv_bfloat16* outh = (__nv_bfloat16*)p.out;
        float gate_keep[16];
        const uint64_t out_policy = l2_evict_first_policy();
        wait_for_predecessor();      // the epilogue reads and writes memory other kernels use

        // The factor of every row of x, if this product scales its rows: a warp adds a row's partial sums of squares in
        // an order that depends on their number alone.  (The swapped form has one tile of x: rows 0 .. M - 1.)
        bool scaled = false;
        if constexpr (kSwapped) {
            scaled = p.scale_sumsq != nullptr;
            if (scaled) {
                constexpr int kWarps = epilogue_warps(kSwapped, BN);
                for (int m = warp - 2; m < p.M && m < BN; m += kWarps) {
                    float sum = 0.0f;
                    for (int g0 = lane; g0 < p.scale_groups; g0 += 32) sum += p.scale_sumsq[(size_t)m * p.scale_groups + g0];
                    sum = warp_sum(sum);
                    if (lane == 0) row_scale[m] = rsqrtf(sum / (float)p.scale_dim + p.scale_eps);
                }
                asm volatile("bar.sync 1, %0;" ::"r"(32 * kWarps) : "memory");      // the epilogue warps only
            }
        }
        const bool emits = kSwapped && p.out_kind == kAddF32 && p.emit_rows != nullptr;
        const int emit_groups = p.N >> 5;
        if (kSwapped && emits && p.splits > 1) {
            int ta, tb, sp;
            decode(blockIdx.x, ta, tb, sp);                   // a split tile is its block's only unit of work
            const int unit = (warp - 2) * p.splits + sp;      // the first (mostly the only) unit of the tile this warp owns
            if (warp - 2 < (BN + p.splits - 1) / p.splits && unit < BN) {
                const int m0 = tb * BN + (unit >> 2) * 4, n = ta * kBM + (unit & 3) * 32 + lane;
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (n < p.N && m0 + e < p.M) x_old[e] = ((const float*)p.out)[(size_t)(m0 + e) * p.N + n];
                have_old = true;
            }
        }

        // What becomes of 16 finished values: row i of the 128-row operand, rows j0 .. j0+15 of the other.
        auto finish = [&](const float (&v)[16], int i, int j0, int c0) {
            if constexpr (!kSwapped) {
                // i is a row m of x, j an output feature n
                finish_rows(v, i, j0, c0, gate_keep, p.out, p.out_kind, p.M, p.N, epilogue_stage, lane, out_policy);
            } else if (p.out_kind == kSwigluBF16) {
                // i is an output feature n, j a row m of x.  Weight rows alternate in runs of 16 (gate rows, then the
                // up rows of the same outputs): lanes 0-15 of a warp hold gate values, lanes 16-31 the matching up values
                const int half_n = p.N >> 1;
                const int o_col = (i >> 5) * 16 + (lane & 15);
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const int m = j0 + c;
                    const float mine = scaled && m < p.M ? v[c] * row_scale[m] : v[c];
                    const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
                    if ((lane & 16) == 0 && i < p.N && m < p.M)
                        outh[(size_t)m * half_n + o_col] = __float2bfloat16_rn(silu_mul(mine, other));
                }
            } else if (emits) {
                // x[m, n] += v, and the updated row goes out as bfloat16 with the sum of its squares over this warp's
                // 32 features (every lane takes part in the sum; a lane past the matrix adds nothing)
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const int m = j0 + c;
                    float sq = 0.0f;
                    if (i < p.N && m < p.M) {
                        const size_t o = (size_t)m * p.N + i;
                        const float xn = outf[o] + v[c];
                        outf[o] = xn;
                        p.emit_rows[o] = __float2bfloat16_rn(xn);
                        sq = xn * xn;
                    }
                    sq = warp_sum(sq);
                    if (lane == 0 && i < p.N && m < p.M) p.emit_sumsq[(size_t)m * emit_groups + (i >> 5)] = sq;
                }
            } else if (i < p.N) {
                // out[m, n]; lanes hold consecutive n
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const int m = j0 + c;
                    if (m < p.M) {
                        const size_t o = (size_t)m * p.N + i;
                        const float val = scaled ? v[c] * row_scale[m] : v[c];
                        if (p.out_kind == kStoreBF16) outh[o] = __float2bfloat16_rn(val);
                        else if (p.out_kind == kAddF32) red_add_f32(outf + o, val);
                        else outf[o] = val;
                    }
                }
            }
        };

        uint32_t acc_it = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x, ++acc_it) {
            int ta, tb, sp;
            decode(u, ta, tb, sp);
            const int kb0 = sp * kb_per_split, kb1 = min(kblocks, kb0 + kb_per_split);
            const int as = acc_it % kAccStages;
            const bool acc_ready = mbar_wait(smem_u32(&acc_full_bar[as]), (acc_it / kAccStages) & 1u, abort_flag, p.error_flag, 104);
            // (a split tile is its block's only unit: every thread of the cluster passes here exactly once)
            if (kSwapped && kRecvInRing && p.splits > 1) cluster_sync_all();
            if (!acc_ready) break;
            tc_fence_after();
            const int i = ta * kBM + quarter * 32 + lane;     // row of the 128-row operand
            const bool empty_range = kb1 <= kb0;              // a split that got no K blocks contributes zeros
            // Split K (swapped form only; `sp` is this block's rank in the cluster of the tile's splits).  The
            // tile is cut into units of four columns (rows m of x) and 32 rows (output features n: a warp's
            // lanes); unit u belongs to the block with rank u % splits, and every block sends its partial
            // of a unit to the owner's receive area, slot [sender][u / splits][lane][4 columns].
            const int units_per_owner = (BN + p.splits - 1) / p.splits;
            const bool pow2 = (p.splits & (p.splits - 1)) == 0;     // the plan's splits are; a forced split may not be
            const int shift = 31 - __clz(p.splits);
            if (!kSwapped) {
                // prompts: the columns go in pairs of 16-column chunks (a gate run and its up run), the pairs
                // alternately to the two warps that share these 32 tensor-memory lanes; both chunks of a pair
                // are read before either is worked on
                const int half = (warp - 2) >> 2;
#pragma unroll 1
                for (int c0 = half * 32; c0 < BN; c0 += 64) {
                    const bool two = c0 + 16 < BN;
                    uint32_t r0[16], r1[16];
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + as * BN + c0, r0);
                    if (two) tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + as * BN + c0 + 16, r1);
                    tmem_ld_wait();
                    float v[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) v[c] = __uint_as_float(r0[c]);
                    finish(v, i, tb * BN + c0, c0);
                    if (two) {
#pragma unroll
                        for (int c = 0; c < 16; ++c) v[c] = __uint_as_float(r1[c]);
                        finish(v, i, tb * BN + c0 + 16, c0 + 16);
                    }
                }
            }
            constexpr int kWarpsPerQuarter = epilogue_warps(kSwapped, BN) / 4;
#pragma unroll 1
            for (int c0 = kSwapped ? ((warp - 2) >> 2) * 16 : BN; c0 < BN; c0 += 16 * kWarpsPerQuarter) {
                uint32_t r[16];
                tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + as * BN + c0, r);
                tmem_ld_wait();
                float v[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) v[c] = empty_range ? 0.0f : __uint_as_float(r[c]);
                if (p.splits > 1) {
#pragma unroll
                    for (int c = 0; c < 16; c += 4) {
                        const int unit = (c0 + c) + quarter;                 // = ((c0 + c) / 4) * 4 + quarter
                        const int owner = pow2 ? (unit & (p.splits - 1)) : unit % p.splits;
                        const int ul = pow2 ? (unit >> shift) : unit / p.splits;
                        const uint32_t slot = recv + (uint32_t)(((sp * units_per_owner + ul) * 32 + lane) * 16);
                        st_cluster_f4(cluster_addr(slot, (uint32_t)owner), v[c], v[c + 1], v[c + 2], v[c + 3]);
                    }
                } else {
                    finish(v, i, tb * BN + c0, c0);
                }
            }
            // the accumulator stage is free again
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty_bar[as]));
        }
    }

    if (kSwapped && kRecvInRing && p.splits > 1 && warp < 2) cluster_sync_all();      // the barrier the epilogue warps pass after the last MMA
    if (kSwapped && p.splits > 1) {
        // The `splits` blocks of a tile form a cluster (rank = split).  Once every block has sent its partials
        // (the cluster barrier makes them visible), each block adds up the units it owns, in rank order
        // whatever the batch, and writes them.  Nothing reads another block's shared memory after the
        // barrier, so the blocks leave without a second one.
        cluster_sync_all();
        if (warp >= 2) {
            int ta, tb, sp;
            decode(blockIdx.x, ta, tb, sp);
            const int units_per_owner = (BN + p.splits - 1) / p.splits;
            float* outf = (float*)p.out;
            __nv_bfloat16* outh = (__nv_bfloat16*)p.out;
#pragma unroll 1
            for (int ul = warp - 2; ul < units_per_owner; ul += epilogue_warps(kSwapped, BN)) {
                const int unit = ul * p.splits + sp;
                if (unit >= BN) break;
                const int m0 = tb * BN + (unit >> 2) * 4, n = ta * kBM + (unit & 3) * 32 + lane;
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int src = 0; src < p.splits; ++src) {
                    const float4 t = ld_shared_f4(recv + (uint32_t)(((src * units_per_owner + ul) * 32 + lane) * 16));
                    a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
                }
                float v[4] = {a.x, a.y, a.z, a.w};
                const bool scaled = p.scale_sumsq != nullptr;
                const bool emits = p.out_kind == kAddF32 && p.emit_rows != nullptr;
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (scaled && m0 + e < p.M) v[e] *= row_scale[m0 + e];
                if (emits) {
                    // (as in the unsplit epilogue: the updated rows as bfloat16 and their squares summed over the warp's 32
                    // features; the four rows' sums go through the shuffles side by side)
                    float sq[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int m = m0 + e;
                        sq[e] = 0.0f;
                        if (n < p.N && m < p.M) {
                            const size_t o = (size_t)m * p.N + n;
                            const float xn = ((have_old && ul == warp - 2) ? x_old[e] : outf[o]) + v[e];
                            outf[o] = xn;
                            p.emit_rows[o] = __float2bfloat16_rn(xn);
                            sq[e] = xn * xn;
                        }
                    }
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) sq[e] += __shfl_xor_sync(0xffffffffu, sq[e], off);
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (lane == 0 && n < p.N && m0 + e < p.M) p.emit_sumsq[(size_t)(m0 + e) * (p.N >> 5) + (n >> 5)] = sq[e];
                    continue;
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int m = m0 + e;
                    if (p.out_kind == kSwigluBF16) {
                        // lanes 0-15 hold gate values, lanes 16-31 the up values of the same outputs
                        const float other = __shfl_xor_sync(0xffffffffu, v[e], 16);
                        if ((lane & 16) == 0 && n < p.N && m < p.M)
                            outh[(size_t)m * (p.N >> 1) + (n >> 5) * 16 + (lane & 15)] = __float2bfloat16_rn(silu_mul(v[e], other));
                    } else if (n < p.N && m < p.M) {
                        const size_t o = (size_t)m * p.N + n;
                        if (p.out_kind == kStoreBF16) outh[o] = __float2bfloat16_rn(v[e]);
                        else if (p.out_kind == kAddF32) red_add_f32(outf + o, v[e]);      // one add per element: the same sum, no load to wait for
                        else outf[o] = v[e];
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- host side ---------------------------------------------------------------------------

// A [rows, K] bfloat16 row-major matrix as tiles of [box_rows, 64] with 128-byte swizzle;
// outside the matrix a tile reads zeros.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    return make_bf16_map(map, base, (uint64_t)rows, (uint64_t)K, (uint64_t)K, box_rows, "gemm_tc");
}

struct Plan {
    bool swapped;
    int bn;
    int splits;
    long cost;      // normal form: waves x the tile's time in the model's units; 0 for the swapped form
};

// The plan is a function of the shape alone.
// Normal form: the grid runs in waves of one block per SM; the narrow tile's width is chosen so that the last
// wave is as full as possible (measured at 2,048 rows, a tile's time hardly depends on its width: about
// 20 + 0.03 x width microseconds at K = 4096).
// Swapped form: up to 128 rows of x always; up to kMaxSwappedRows rows (one tile of 256 rows of x) when the
// normal form would leave SMs without a tile, i.e. against a narrow weight matrix: a tile's K loop of 26 us
// would then bound the product, while here every weight tile is streamed once and K is split over the SMs.
// The split aims at a block (two for narrow tiles) on every SM and keeps at least four K blocks per block.
static Plan make_plan(int M, int N, int K, int sm_count, int force_splits = 0, bool gate_runs = false) {
    Plan pl;
    pl.swapped = false;
    pl.bn = 128;
    pl.splits = 1;
    pl.cost = 0;
    long normal_tiles = (long)((M + kBM - 1) / kBM) * ((N + 127) / 128);
    if (N >= 192) {
        const int tiles_m = (M + kBM - 1) / kBM;
        long best = -1;
        for (int bn : {256, 240, 224, 208, 192}) {
            if (gate_runs && bn % 32 != 0) continue;      // a tile must hold whole pairs of gate and up runs
            const long tiles = (long)tiles_m * ((N + bn - 1) / bn);
            const long cost = ((tiles + sm_count - 1) / sm_count) * (2000 + 3 * bn);
            if (best < 0 || cost < best) { best = cost; pl.bn = bn; normal_tiles = tiles; }
        }
        pl.cost = best;
    }
    if (M <= 128 || (M <= kMaxSwappedRows && normal_tiles < sm_count)) {
        pl.swapped = true;
        pl.bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
        const int tiles = (N + kBM - 1) / kBM;
        const int kblocks = (K + kBK - 1) / kBK;
        const int slots = sm_count * (pl.bn <= 128 ? 2 : 1);
        int s = slots / tiles;
        if (s > kblocks / 4) s = kblocks / 4;
        if (s > kMaxSplits) s = kMaxSplits;
        // the splits of a tile are one cluster: sizes 2, 4, 8 are placed well, odd sizes were measured slower
        int pow2 = 1;
        while (pow2 * 2 <= s) pow2 *= 2;
        s = pow2;
        if (force_splits > 0) s = force_splits > kMaxSplits ? kMaxSplits : force_splits;
        if (s > kblocks) s = kblocks;
        if (s < 1) s = 1;
        pl.splits = s;
    }
    return pl;
}

template <int BN, bool kSwapped>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int sm_count, cudaStream_t stream) {
    constexpr int stages = stages_for<BN>(kSwapped);
    const size_t smem = (size_t)stages * (kBM * kBK * 2 + BN * kBK * 2) + (kSwapped ? (BN < 128 ? BN * 512 + 4096 : 0) : 8 * kEpilogueStageBytes) + 1024;      // ring, split-K receive area behind it, alignment
    auto kernel = gemm_tc_kernel<BN, kSwapped>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles_a = (p.rows_a + kBM - 1) / kBM, tiles_b = (p.rows_b + BN - 1) / BN;
    const int units = tiles_a * tiles_b * p.splits;
    const int per_sm = (kSwapped && BN <= 128) ? 2 : 1;
    // split K: one block per (tile, split), the splits of a tile being one cluster; else a persistent grid
    const int grid = p.splits > 1 ? units : (units < sm_count * per_sm ? units : sm_count * per_sm);
    launch_kernel_clustered(kernel, grid, threads_for(kSwapped, BN), smem, p.splits > 1 ? p.splits : 1, stream, ma, mb, p);
    return CITLALI_LAUNCH_CHECK();
}

}  // namespace tc
}  // namespace citlali

using namespace citlali;
using namespace citlali::tc;

// > 0: from this many rows of x on, the product runs on pairs of SMs where that fills the device's waves no
// worse. Measured on Qwen3-8B's four projections at 256 to 8,192 rows: with equal waves the pair kernel takes
// 0.92-0.97 of the one-block kernel's time (0.82 at 8,192 rows), and it loses where its 256-row tiles of one
// width need a wave more; below 512 rows it never won.
static int g_pair_rows = 512;

// Sets the threshold and returns the one that stood before.
extern "C" int citlali_gemm_tc_set_pair_rows(int rows) {
    const int before = g_pair_rows;
    g_pair_rows = rows;
    return before;
}

// Whether the pair kernel takes this product: a normal-form plan, enough rows, and waves of pairs that cost
// less than 0.95 of the one-block waves in the plan's own model.
static bool runs_on_pairs(int M, int N, int K, const Plan& pl) {
    if (pl.swapped || pl.cost <= 0 || g_pair_rows <= 0 || M < g_pair_rows) return false;
    int bn = 0, pairs = 0;
    citlali_gemm_tc_pair_plan(M, N, K, &bn, &pairs);
    if (pairs <= 0) return false;
    const long units = (long)((M + 2 * kBM - 1) / (2 * kBM)) * ((N + bn - 1) / bn);
    const long pair_cost = ((units + pairs - 1) / pairs) * (2000 + 3 * bn);
    return pair_cost * 95 < pl.cost * 100;
}

extern "C" int citlali_gemm_tc_runs_on_pairs(int M, int N, int K, int sm_count, int gate_runs) {
    if (sm_count <= 0) sm_count = device_sm_count();
    return runs_on_pairs(M, N, K, make_plan(M, N, K, sm_count, 0, gate_runs != 0)) ? 1 : 0;
}

// The bounded wait of the tensor-core kernels, on its own: one block waits on an mbarrier on which nothing ever
// arrives, with `limit_ns` instead of the kernels' two seconds.  The wait gives up, records code 900 and the
// block in error_flag[1..2] and raises the block's abort word, which the other threads see; the kernel then
// leaves normally.  result[0] = what the wait returned (0), result[1] = the abort word as thread 32 saw it.
__global__ void wait_selftest_kernel(int32_t* error_flag, unsigned long long limit_ns, int* result) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;
    if (threadIdx.x == 0) {
        abort_word = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_barrier_init();
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait(smem_u32(&bar), 0, abort_flag, error_flag, 900, limit_ns);
    __syncthreads();
    if (threadIdx.x == 0) result[0] = ok ? 1 : 0;
    if (threadIdx.x == 32) result[1] = *abort_flag;
}

extern "C" int citlali_wait_selftest(int32_t* error_flag, int* result, long long limit_ns, cudaStream_t stream) {
    if (limit_ns < 0 || limit_ns > 1000000000ll) {
        set_last_error("wait_selftest: the limit must lie between 0 and one second");
        return kBadShape;
    }
    wait_selftest_kernel<<<1, 64, 0, stream>>>(error_flag, (unsigned long long)limit_ns, result);
    return CITLALI_LAUNCH_CHECK();
}

// How the product of this shape would run: *swapped, *bn and the K split (*splits).
extern "C" int citlali_gemm_tc_plan(int M, int N, int K, int sm_count, int force_splits, int* swapped, int* bn, int* splits) {
    if (sm_count <= 0) sm_count = device_sm_count();
    Plan pl = make_plan(M, N, K, sm_count, force_splits);
    if (swapped) *swapped = pl.swapped;
    if (bn) *bn = pl.bn;
    if (splits) *splits = pl.splits;
    return 0;
}

// y = x . w^T with x [M, K] and w [N, K] bfloat16, contiguous, 16-byte aligned, K a multiple of 8.
// `mode` bits: 1 = y (float32 [M, N]) += product; 2 = SiLU-gate epilogue: w's rows alternate in runs
// of 16 between gate and up rows and y is bfloat16 [M, N/2] = silu(gate) * up (N a multiple of 32).
// Without them y is [M, N] of y_dtype (0 float32, 1 bfloat16).  A shape that splits K (few rows, see
// citlali_gemm_tc_plan) runs the splits of a tile as one thread-block cluster whose blocks add their
// partial sums through distributed shared memory in split order; it needs no scratch memory.
// `force_splits` > 0 replaces the plan's K split (for tuning and tests; at most 8).
extern "C" int citlali_gemm_tc(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                               int mode, int force_splits, int32_t* error_flag, int sm_count, cudaStream_t stream) {
    return citlali_gemm_tc_normed(x, w, y, y_dtype, M, N, K, mode, force_splits, error_flag, sm_count, nullptr, nullptr,
                                  nullptr, 0, 0, 0.0f, stream);
}

// citlali_gemm_tc for few rows of x (the form with the weights as the 128-row operand: see citlali_gemm_tc_plan) with a
// layer norm's work in its epilogue.  `emit_rows` / `emit_sumsq` (both or neither; mode bit 0, N a multiple of 32): the
// product is added to the float32 rows y as always, and the updated rows also go out as bfloat16 [M, N] with the sums of
// their squares over each 32 consecutive features, float32 [M, N / 32].  `scale_sumsq` (float32 [M, scale_groups], the
// sums of squares of the rows of x over groups of features): every result row m is multiplied by
// rsqrt(sum of its groups / scale_dim + scale_eps) before it is stored, gated or added.
extern "C" int citlali_gemm_tc_normed(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                                      int mode, int force_splits, int32_t* error_flag, int sm_count,
                                      void* emit_rows, float* emit_sumsq, const float* scale_sumsq, int scale_groups,
                                      int scale_dim, float scale_eps, cudaStream_t stream) {
    const bool accumulate = (mode & 1) != 0, swiglu = (mode & 2) != 0;
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0) {
        set_last_error("gemm_tc: the inner size %d must be a positive multiple of 8 (rows of 16-byte multiples for TMA)", K);
        return kBadShape;
    }
    if (((uintptr_t)x | (uintptr_t)w) & 15u) {
        set_last_error("gemm_tc: operands must start on 16-byte boundaries");
        return kBadAlignment;
    }
    if (accumulate && y_dtype != kF32) {
        set_last_error("gemm_tc: accumulation needs a float32 output");
        return kBadDType;
    }
    if (y_dtype != kF32 && y_dtype != kBF16) {
        set_last_error("gemm_tc: output dtype code %d is neither float32 nor bfloat16", y_dtype);
        return kBadDType;
    }
    if (swiglu && (accumulate || y_dtype != kBF16 || N % 32 != 0)) {
        set_last_error("gemm_tc: the gate epilogue needs a bfloat16 output and N a multiple of 32 (N %d)", N);
        return kBadShape;
    }
    if (sm_count <= 0) sm_count = device_sm_count();
    const Plan pl = make_plan(M, N, K, sm_count, force_splits, swiglu);
    const bool normed = emit_rows != nullptr || emit_sumsq != nullptr || scale_sumsq != nullptr;
    if (normed) {
        if (!pl.swapped) {
            set_last_error("gemm_tc_normed: %d rows of x run the prompt form of the product, whose epilogue does no norm work", M);
            return kBadShape;
        }
        if ((emit_rows == nullptr) != (emit_sumsq == nullptr) || (emit_rows != nullptr && (!accumulate || N % 32 != 0))) {
            set_last_error("gemm_tc_normed: emitting needs both outputs, the adding mode and N a multiple of 32 (N %d)", N);
            return kBadShape;
        }
        if (scale_sumsq != nullptr && (scale_groups <= 0 || scale_dim <= 0)) {
            set_last_error("gemm_tc_normed: scaling needs the number of groups and the norm's width");
            return kBadShape;
        }
    }
    if (runs_on_pairs(M, N, K, pl)) return citlali_gemm_tc_pair(x, w, y, y_dtype, M, N, K, mode, error_flag, stream);
    GemmParams p;
    p.emit_rows = (__nv_bfloat16*)emit_rows; p.emit_sumsq = emit_sumsq;
    p.scale_sumsq = scale_sumsq; p.scale_groups = scale_groups; p.scale_dim = scale_dim; p.scale_eps = scale_eps;
    p.M = M; p.N = N; p.K = K;
    p.splits = pl.splits;
    p.error_flag = error_flag;
    p.out = y;
    p.out_kind = swiglu ? kSwigluBF16 : accumulate ? kAddF32 : (y_dtype == kF32 ? kStoreF32 : kStoreBF16);
    p.rows_a = pl.swapped ? N : M;
    p.rows_b = pl.swapped ? M : N;
    CUtensorMap ma, mb;
    int rc;
    if (pl.swapped) {
        if ((rc = make_map(&ma, w, N, K, kBM))) return rc;
        if ((rc = make_map(&mb, x, M, K, pl.bn))) return rc;
        switch (pl.bn) {
            case 16: rc = launch<16, true>(ma, mb, p, sm_count, stream); break;
            case 32: rc = launch<32, true>(ma, mb, p, sm_count, stream); break;
            case 64: rc = launch<64, true>(ma, mb, p, sm_count, stream); break;
            case 128: rc = launch<128, true>(ma, mb, p, sm_count, stream); break;
            default: rc = launch<256, true>(ma, mb, p, sm_count, stream); break;
        }
    } else {
        if ((rc = make_map(&ma, x, M, K, kBM))) return rc;
        if ((rc = make_map(&mb, w, N, K, pl.bn))) return rc;
        switch (pl.bn) {
            case 256: rc = launch<256, false>(ma, mb, p, sm_count, stream); break;
            case 240: rc = launch<240, false>(ma, mb, p, sm_count, stream); break;
            case 224: rc = launch<224, false>(ma, mb, p, sm_count, stream); break;
            case 208: rc = launch<208, false>(ma, mb, p, sm_count, stream); break;
            case 192: rc = launch<192, false>(ma, mb, p, sm_count, stream); break;
            default: rc = launch<128, false>(ma, mb, p, sm_count, stream); break;
        }
    }
    return rc;
}
