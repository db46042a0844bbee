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
// several blocks so that every SM streams weights, each writing a float32 partial, and a second
// kernel adds the partials in split order.  The split depends on the shape alone, never on the
// batch, so a row's result does not depend on what else is in the step.
//
// Every wait on an mbarrier gives up after a time limit, raises the error word and makes the
// block leave through the normal exit (TMEM freed, copies in flight awaited).
#include "api.h"
#include "common.cuh"
#include "tc_common.cuh"

#include <cstdio>
#include <map>
#include <mutex>
#include <tuple>

namespace citlali {
namespace tc {

constexpr int kBM = 128, kBK = 64, kAccStages = 2;
constexpr int kThreads = 192;

enum OutKind : int { kStoreBF16 = 0, kStoreF32 = 1, kAddF32 = 2, kPartialF32 = 3 };

struct GemmParams {
    void* out;             // [M, N] (or the partials' workspace [splits, M, N])
    int out_kind;
    int M, N, K;           // the product's logical shape: y[M, N] = x[M, K] w[N, K]^T
    int rows_a, rows_b;    // rows of the 128-row operand and of the BN-row operand
    int splits;            // K is cut into this many ranges of whole 64-blocks
    int32_t* error_flag;
};

template <int BN>
constexpr int stages_for(bool swapped) {
    // swapped (decoding): two blocks per SM, about 100 KB each; normal: one block of 192 KB
    return swapped ? (BN <= 16 ? 6 : BN <= 32 ? 5 : BN <= 64 ? 4 : 6) : (BN <= 128 ? 6 : 4);
}

template <int BN, bool kSwapped>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmParams p) {
    constexpr int kStages = stages_for<BN>(kSwapped);
    constexpr uint32_t kBytesA = kBM * kBK * 2, kBytesB = BN * kBK * 2;
    constexpr uint32_t kTmemCols = (kAccStages * BN) < 32 ? 32 : (kAccStages * BN);
    constexpr uint32_t kIdesc = instr_desc_bf16(kBM, BN);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], acc_full_bar[kAccStages], acc_empty_bar[kAccStages];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;            // tile storage starts on a 1024-byte boundary
    const uint32_t smem_a = tiles, smem_b = tiles + kStages * kBytesA;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        abort_word = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int a = 0; a < kAccStages; ++a) { mbar_init(smem_u32(&acc_full_bar[a]), 1); mbar_init(smem_u32(&acc_empty_bar[a]), 4); }
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

    // unit -> (a tile, b tile, split).  Normal: the x tile index runs fastest, so blocks that run
    // together share a weight tile.  Swapped: the split runs fastest, then the weight tile.
    auto decode = [&](int u, int& ta, int& tb, int& sp) {
        if (kSwapped) { sp = u % p.splits; u /= p.splits; ta = u % tiles_a; tb = u / tiles_a; }
        else { sp = u % p.splits; u /= p.splits; ta = u % tiles_a; tb = u / tiles_a; }
    };

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
                int ta, tb, sp;
                decode(u, ta, tb, sp);
                const int kb0 = sp * kb_per_split, kb1 = min(kblocks, kb0 + kb_per_split);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / kStages) & 1u) ^ 1u, abort_flag, p.error_flag, 101)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full_bar[s]);
                    mbar_arrive_expect_tx(bar, kBytesA + kBytesB);
                    tma_load_2d(smem_a + s * kBytesA, &map_a, kb * kBK, ta * kBM, bar);
                    tma_load_2d(smem_b + s * kBytesB, &map_b, kb * kBK, tb * BN, bar);
                }
            }
            if (!ok) {
                // leaving early: let the copies this thread issued land before shared memory goes away
                const uint32_t first = it > (uint32_t)kStages ? it - kStages : 0u;
                for (uint32_t j = first; j < it; ++j) {
                    const uint32_t bar = smem_u32(&full_bar[j % kStages]);
                    const uint64_t start = global_timer();
                    while (!mbar_try_wait(bar, (j / kStages) & 1u) && global_timer() - start < 100000000ull) {}
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, acc_it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++acc_it) {
                int ta, tb, sp;
                decode(u, ta, tb, sp);
                const int kb0 = sp * kb_per_split, kb1 = min(kblocks, kb0 + kb_per_split);
                const int as = acc_it % kAccStages;
                if (!mbar_wait(smem_u32(&acc_empty_bar[as]), ((acc_it / kAccStages) & 1u) ^ 1u, abort_flag, p.error_flag, 102)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + as * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(smem_u32(&full_bar[s]), (it / kStages) & 1u, abort_flag, p.error_flag, 103)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        mma_bf16(tmem_d, smem_desc_sw128(smem_a + s * kBytesA, k * 32), smem_desc_sw128(smem_b + s * kBytesB, k * 32),
                                 kIdesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    mma_commit(smem_u32(&empty_bar[s]));
                }
                if (ok) mma_commit(smem_u32(&acc_full_bar[as]));
            }
        }
        __syncwarp();
    } else {
        const int quarter = warp & 3;                       // the TMEM lanes this warp may read: 32 * quarter ..
        uint32_t acc_it = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x, ++acc_it) {
            int ta, tb, sp;
            decode(u, ta, tb, sp);
            const int kb0 = sp * kb_per_split, kb1 = min(kblocks, kb0 + kb_per_split);
            const int as = acc_it % kAccStages;
            if (!mbar_wait(smem_u32(&acc_full_bar[as]), (acc_it / kAccStages) & 1u, abort_flag, p.error_flag, 104)) break;
            tc_fence_after();
            const int i = ta * kBM + quarter * 32 + lane;     // row of the 128-row operand
            const bool empty_range = kb1 <= kb0;              // a split that got no K blocks contributes zeros
            float* outf = (float*)p.out;
            __nv_bfloat16* outh = (__nv_bfloat16*)p.out;
            if (p.out_kind == kPartialF32) outf += (size_t)sp * p.M * p.N;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + as * BN + c0, r);
                tmem_ld_wait();
                if (empty_range) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) r[c] = 0u;
                }
                const int j0 = tb * BN + c0;                  // first row of the BN-row operand in this chunk
                if (kSwapped) {
                    // i is an output feature n, j a row m of x: out[m, n]; lanes hold consecutive n
                    if (i < p.N) {
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int m = j0 + c;
                            if (m < p.M) {
                                const size_t o = (size_t)m * p.N + i;
                                const float v = __uint_as_float(r[c]);
                                if (p.out_kind == kStoreBF16) outh[o] = __float2bfloat16_rn(v);
                                else if (p.out_kind == kAddF32) outf[o] += v;
                                else outf[o] = v;
                            }
                        }
                    }
                } else {
                    // i is a row m of x, j an output feature n: this thread holds 16 consecutive n
                    if (i < p.M && j0 < p.N) {
                        const size_t o = (size_t)i * p.N + j0;
                        const bool full = j0 + 16 <= p.N;
                        if (p.out_kind == kStoreBF16) {
                            if (full && (p.N % 8) == 0) {
                                uint32_t w[8];
#pragma unroll
                                for (int c = 0; c < 8; ++c) {
                                    __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[2 * c]), __uint_as_float(r[2 * c + 1]));
                                    w[c] = *reinterpret_cast<uint32_t*>(&h2);
                                }
                                uint4* dst = reinterpret_cast<uint4*>(outh + o);
                                dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                                dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
                            } else {
                                for (int c = 0; c < 16 && j0 + c < p.N; ++c) outh[o + c] = __float2bfloat16_rn(__uint_as_float(r[c]));
                            }
                        } else if (full && (p.N % 4) == 0) {
                            float4* dst = reinterpret_cast<float4*>(outf + o);
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                float4 v = make_float4(__uint_as_float(r[4 * c]), __uint_as_float(r[4 * c + 1]),
                                                       __uint_as_float(r[4 * c + 2]), __uint_as_float(r[4 * c + 3]));
                                if (p.out_kind == kAddF32) {
                                    const float4 old = dst[c];
                                    v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
                                }
                                dst[c] = v;
                            }
                        } else {
                            for (int c = 0; c < 16 && j0 + c < p.N; ++c) {
                                const float v = __uint_as_float(r[c]);
                                if (p.out_kind == kAddF32) outf[o + c] += v; else outf[o + c] = v;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty_bar[as]));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// out (+)= sum over splits of partials, in split order.
__global__ void splitk_reduce_kernel(const float* __restrict__ partials, void* __restrict__ out, int out_kind,
                                     size_t elements, int splits) {
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= elements) return;
    float s = partials[e];
    for (int z = 1; z < splits; ++z) s += partials[(size_t)z * elements + e];
    if (out_kind == kStoreBF16) ((__nv_bfloat16*)out)[e] = __float2bfloat16_rn(s);
    else if (out_kind == kAddF32) ((float*)out)[e] += s;
    else ((float*)out)[e] = s;
}

// ---- host side ---------------------------------------------------------------------------

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

// A [rows, K] bfloat16 row-major matrix as tiles of [box_rows, 64] with 128-byte swizzle;
// outside the matrix a tile reads zeros.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_last_error("gemm_tc: the driver does not provide cuTensorMapEncodeTiled");
        return kNoDriverEntry;
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("gemm_tc: cuTensorMapEncodeTiled failed with %d for a [%d, %d] matrix at %p", (int)r, rows, K, base);
        return kBadShape;
    }
    return 0;
}

struct Plan {
    bool swapped;
    int bn;
    int splits;
};

// The plan is a function of the shape alone.  Swapped up to 128 rows of x; the split aims at
// two blocks on every SM and keeps at least four K blocks per block.
static Plan make_plan(int M, int N, int K, int sm_count) {
    Plan pl;
    pl.swapped = M <= 128;
    if (pl.swapped) {
        pl.bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
        const int tiles = (N + kBM - 1) / kBM;
        const int kblocks = (K + kBK - 1) / kBK;
        const int slots = sm_count * (pl.bn <= 64 ? 2 : 1);
        int s = slots / tiles;
        if (s > kblocks / 4) s = kblocks / 4;
        if (s > 16) s = 16;
        if (s < 1) s = 1;
        pl.splits = s;
    } else {
        pl.bn = N >= 256 ? 256 : 128;
        pl.splits = 1;
    }
    return pl;
}

template <int BN, bool kSwapped>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int sm_count, cudaStream_t stream) {
    constexpr int stages = stages_for<BN>(kSwapped);
    const size_t smem = (size_t)stages * (kBM * kBK * 2 + BN * kBK * 2) + 1024;
    auto kernel = gemm_tc_kernel<BN, kSwapped>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles_a = (p.rows_a + kBM - 1) / kBM, tiles_b = (p.rows_b + BN - 1) / BN;
    const int units = tiles_a * tiles_b * p.splits;
    const int per_sm = (kSwapped && BN <= 64) ? 2 : 1;
    const int grid = units < sm_count * per_sm ? units : sm_count * per_sm;
    kernel<<<grid, kThreads, smem, stream>>>(ma, mb, p);
    return CITLALI_LAUNCH_CHECK();
}

}  // namespace tc
}  // namespace citlali

using namespace citlali;
using namespace citlali::tc;

// How the product of this shape would run: *swapped, *bn, *splits, and the bytes of float32
// scratch it needs for split-K partials (0 if it does not split).
extern "C" int citlali_gemm_tc_plan(int M, int N, int K, int sm_count, int* swapped, int* bn, int* splits,
                                    size_t* workspace_bytes) {
    Plan pl = make_plan(M, N, K, sm_count);
    if (swapped) *swapped = pl.swapped;
    if (bn) *bn = pl.bn;
    if (splits) *splits = pl.splits;
    if (workspace_bytes) *workspace_bytes = pl.splits > 1 ? (size_t)pl.splits * M * N * sizeof(float) : 0;
    return 0;
}

// y[M, N] (y_dtype: 0 float32, 1 bfloat16) = x . w^T, or with accumulate != 0: y (float32) += x . w^T.
// x [M, K] and w [N, K] are bfloat16, contiguous, 16-byte aligned, K a multiple of 8.
// `workspace` must hold what citlali_gemm_tc_plan reports for this shape.
extern "C" int citlali_gemm_tc(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                               int accumulate, void* workspace, size_t workspace_bytes, int32_t* error_flag,
                               int sm_count, cudaStream_t stream) {
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
    if (sm_count <= 0) sm_count = 148;
    const Plan pl = make_plan(M, N, K, sm_count);
    const int final_kind = accumulate ? kAddF32 : (y_dtype == kF32 ? kStoreF32 : kStoreBF16);
    GemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.splits = pl.splits;
    p.error_flag = error_flag;
    if (pl.splits > 1) {
        const size_t need = (size_t)pl.splits * M * N * sizeof(float);
        if (workspace == nullptr || workspace_bytes < need) {
            set_last_error("gemm_tc: a [%d, %d, %d] product splits K %d ways and needs %zu bytes of scratch, %zu were given",
                           M, N, K, pl.splits, need, workspace_bytes);
            return kTooLarge;
        }
        p.out = workspace;
        p.out_kind = kPartialF32;
    } else {
        p.out = y;
        p.out_kind = final_kind;
    }
    CUtensorMap ma, mb;
    int rc;
    if (pl.swapped) {
        p.rows_a = N; p.rows_b = M;
        if ((rc = make_map(&ma, w, N, K, kBM))) return rc;
        if ((rc = make_map(&mb, x, M, K, pl.bn))) return rc;
        switch (pl.bn) {
            case 16: rc = launch<16, true>(ma, mb, p, sm_count, stream); break;
            case 32: rc = launch<32, true>(ma, mb, p, sm_count, stream); break;
            case 64: rc = launch<64, true>(ma, mb, p, sm_count, stream); break;
            default: rc = launch<128, true>(ma, mb, p, sm_count, stream); break;
        }
    } else {
        p.rows_a = M; p.rows_b = N;
        if ((rc = make_map(&ma, x, M, K, kBM))) return rc;
        if ((rc = make_map(&mb, w, N, K, pl.bn))) return rc;
        if (pl.bn == 256) rc = launch<256, false>(ma, mb, p, sm_count, stream);
        else rc = launch<128, false>(ma, mb, p, sm_count, stream);
    }
    if (rc) return rc;
    if (pl.splits > 1) {
        const size_t elements = (size_t)M * N;
        splitk_reduce_kernel<<<(unsigned)((elements + 255) / 256), 256, 0, stream>>>((const float*)workspace, y, final_kind,
                                                                                    elements, pl.splits);
        return CITLALI_LAUNCH_CHECK();
    }
    return 0;
}
