// y[M, N] = x[M, K] . w[N, K]^T in bfloat16 for many rows of x (prompts), with two SMs on one tile.
//
// The blocks of a cluster of two share [256 x BN] output tiles: tcgen05.mma with cta_group::2, issued
// by the block with cluster rank 0, multiplies 256 rows of x (128 from each block's shared memory)
// by BN rows of w (BN / 2 from each block's shared memory) into the tensor memory of both blocks,
// each holding its 128 rows of the accumulator.  Per K block a block therefore fetches 128 rows of x
// and only half of the weight tile, which is what bounds the one-block kernel: its shared memory
// takes the TMA writes and feeds the tensor core's reads of both whole operands.
// Roles in each block (as in the one-block kernel):
//   warp 0, one lane: TMA producer of this block's halves.  The bytes of both blocks are counted on
//                     the full barrier of the block with rank 0; neither load is multicast.
//   warp 1:           allocates tensor memory (both blocks, together); in the block with rank 0 one
//                     lane issues the MMAs; tcgen05.commit arrives on the barriers of both blocks.
//   warps 2-9:        epilogue of this block's 128 rows (two warps share 32 tensor-memory lanes and take
//                     alternate pairs of 16-column chunks; values leave through shared memory so that every
//                     store covers whole sectors); the accumulator stage is handed back on a
//                     barrier of the block with rank 0 on which the warps of both blocks arrive.
// Every wait on an mbarrier gives up after a time limit, raises the error word and makes the block
// leave through the normal exit (cluster barrier, tensor memory freed).
#include "api.h"
#include "common.cuh"
#include "tc_common.cuh"
#include "tc_host.h"

namespace citlali {
namespace tc {
namespace pair {

constexpr int kBM = 128, kBK = 64, kAccStages = 2;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr uint32_t kTmemCols = 512;

struct Params {
    void* out;
    int out_kind;
    int M, N, K;
    int32_t* error_flag;
    int band;              // row tiles that are finished across all weight tiles before the next ones begin
};

template <int BN>
constexpr int stages_for() { return BN <= 192 ? 7 : 6; }      // 16 KB of x and BN * 64 bytes of w a stage

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, Params p) {
    constexpr int kStages = stages_for<BN>();
    constexpr uint32_t kBytesA = kBM * kBK * 2, kBytesB = (BN / 2) * kBK * 2;
    constexpr uint32_t kIdesc = instr_desc_bf16(2 * kBM, BN);

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], acc_full_bar[kAccStages], acc_empty_bar[kAccStages];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;

    dependents_may_launch();
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;            // tile storage starts on a 1024-byte boundary
    const uint32_t smem_a = tiles, smem_b = tiles + kStages * kBytesA;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t epilogue_stage = tiles + kStages * (kBytesA + kBytesB) + (uint32_t)((warp - 2) & 7) * kEpilogueStageBytes;
    const uint32_t rank = cluster_rank();                     // 0 issues the MMAs
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        abort_word = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int a = 0; a < kAccStages; ++a) { mbar_init(smem_u32(&acc_full_bar[a]), 1); mbar_init(smem_u32(&acc_empty_bar[a]), 2 * kEpilogueWarps); }
        fence_barrier_init();
        fence_async_proxy();
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                       // both blocks' barriers exist before either is signalled
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int tiles_m = (p.M + 2 * kBM - 1) / (2 * kBM), tiles_n = (p.N + BN - 1) / BN;
    const int kblocks = (p.K + kBK - 1) / kBK;
    const int units = tiles_m * tiles_n;
    const int pair_id = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    // unit -> (row tile, weight tile): the row tile runs fastest, so pairs that run together share a weight tile.  Of a
    // matrix of many rows (several prompts in a step) the row tiles are taken in bands of p.band: a band's rows of x
    // are few enough to stay in L2 while all the weight tiles pass by, so x comes from memory once and the weights once
    // a band; without bands every weight tile would bring all of x in again.
    const int per_band = p.band * tiles_n;
    auto unit_tiles = [&](int u, int& tm, int& tn) {
        const int b = u / per_band, r = u - b * per_band;
        const int rows_here = min(p.band, tiles_m - b * p.band);
        tn = r / rows_here;
        tm = b * p.band + (r - tn * rows_here);
    };

    if (warp == 0) {
        if (lane == 0) {
            wait_for_predecessor();
            const uint32_t leader_full0 = cluster_addr(smem_u32(&full_bar[0]), 0);
            uint32_t it = 0;
            bool ok = true;
            for (int u = pair_id; u < units && ok; u += pairs) {
                int tm, tn;
                unit_tiles(u, tm, tn);
                const int row_a = tm * 2 * kBM + (int)rank * kBM, row_b = tn * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / kStages) & 1u) ^ 1u, abort_flag, p.error_flag, 301)) { ok = false; break; }
                    if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[s]), 2 * (kBytesA + kBytesB));
                    const uint32_t bar = leader_full0 + (uint32_t)s * 8u;
                    tma_load_2d_pair(smem_a + s * kBytesA, &map_a, kb * kBK, row_a, bar);
                    tma_load_2d_pair(smem_b + s * kBytesB, &map_b, kb * kBK, row_b, bar);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // as in the one-block kernel: stage and phase are counted, descriptors made by addition, and the next
            // stage's barrier is looked up before the current MMAs are issued
            uint32_t acc_it = 0, stage = 0, phase = 0;
            const uint64_t desc_a0 = smem_desc_sw128(smem_a, 0), desc_b0 = smem_desc_sw128(smem_b, 0);
            const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
            bool ok = true;
            for (int u = pair_id; u < units && ok; u += pairs, ++acc_it) {
                const int as = acc_it % kAccStages;
                if (!mbar_wait(smem_u32(&acc_empty_bar[as]), ((acc_it / kAccStages) & 1u) ^ 1u, abort_flag, p.error_flag, 302)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + as * BN;
                uint32_t accumulate = 0;
                bool landed = kblocks > 0 && mbar_try_wait(full0 + stage * 8u, phase);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!landed && !mbar_wait(full0 + stage * 8u, phase, abort_flag, p.error_flag, 303)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t da = desc_a0 + (uint64_t)(stage * (kBytesA >> 4)), db = desc_b0 + (uint64_t)(stage * (kBytesB >> 4));
                    const uint32_t this_empty = empty0 + stage * 8u;
                    if (++stage == (uint32_t)kStages) { stage = 0; phase ^= 1u; }
                    landed = kb + 1 < kblocks && mbar_try_wait(full0 + stage * 8u, phase);
                    mma_bf16_pair(tmem_d, da, db, kIdesc, accumulate);
                    mma_bf16_pair(tmem_d, da + 2, db + 2, kIdesc, 1u);
                    mma_bf16_pair(tmem_d, da + 4, db + 4, kIdesc, 1u);
                    mma_bf16_pair(tmem_d, da + 6, db + 6, kIdesc, 1u);
                    mma_commit_pair(this_empty, 3);
                    accumulate = 1u;
                }
                if (ok) mma_commit_pair(smem_u32(&acc_full_bar[as]), 3);
            }
        }
        __syncwarp();
    } else {
        const int quarter = warp & 3;                       // the TMEM lanes this warp may read: 32 * quarter ..
        float gate_keep[16];
        const uint64_t out_policy = l2_evict_first_policy();
        wait_for_predecessor();      // the epilogue reads and writes memory other kernels use

        auto finish = [&](const float (&v)[16], int i, int j0, int c0) {
            finish_rows(v, i, j0, c0, gate_keep, p.out, p.out_kind, p.M, p.N, epilogue_stage, lane, out_policy);
        };

        const uint32_t leader_acc_empty0 = cluster_addr(smem_u32(&acc_empty_bar[0]), 0);
        uint32_t acc_it = 0;
        for (int u = pair_id; u < units; u += pairs, ++acc_it) {
            int tm, tn;
            unit_tiles(u, tm, tn);
            const int as = acc_it % kAccStages;
            if (!mbar_wait(smem_u32(&acc_full_bar[as]), (acc_it / kAccStages) & 1u, abort_flag, p.error_flag, 304)) break;
            tc_fence_after();
            const int i = tm * 2 * kBM + (int)rank * kBM + quarter * 32 + lane;     // row of x
            const int half = (warp - 2) >> 2;
#pragma unroll 1
            for (int c0 = half * 32; c0 < BN; c0 += 64) {
                uint32_t r0[16], r1[16];
                tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + as * BN + c0, r0);
                tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + as * BN + c0 + 16, r1);
                tmem_ld_wait();
                float v[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) v[c] = __uint_as_float(r0[c]);
                finish(v, i, tn * BN + c0, c0);
#pragma unroll
                for (int c = 0; c < 16; ++c) v[c] = __uint_as_float(r1[c]);
                finish(v, i, tn * BN + c0 + 16, c0 + 16);
            }
            // the accumulator stage is free again: all eight epilogue warps of the pair say so to rank 0
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + (uint32_t)as * 8u);
        }
    }

    // Both blocks stay until neither has loads, MMAs or arrivals in flight that touch the other.
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// A [rows, K] bfloat16 row-major matrix as tiles of [box_rows, 64] with 128-byte swizzle;
// outside the matrix a tile reads zeros.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    return make_bf16_map(map, base, (uint64_t)rows, (uint64_t)K, (uint64_t)K, box_rows, "gemm_tc_pair");
}

// The number of clusters of two that the device runs at once (not every SM has a partner free).
template <int BN>
static int resident_pairs(size_t smem) {
    static int cached = -1;
    if (cached >= 0) return cached;
    if (cudaFuncSetAttribute(gemm_tc_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * device_sm_count());
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<BN>, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = 0;
    }
    cached = n;
    return n;
}

template <int BN>
static int launch(const void* x, const void* w, const Params& p, cudaStream_t stream) {
    constexpr int stages = stages_for<BN>();
    const size_t smem = (size_t)stages * (kBM * kBK * 2 + (BN / 2) * kBK * 2) + kEpilogueWarps * kEpilogueStageBytes + 1024;
    auto kernel = gemm_tc_pair_kernel<BN>;
    const int pairs_max = resident_pairs<BN>(smem);
    if (pairs_max <= 0) {
        set_last_error("gemm_tc_pair: the device runs no cluster of two blocks with %zu bytes of shared memory", smem);
        return kTooLarge;
    }
    CUtensorMap ma, mb;
    int rc;
    if ((rc = make_map(&ma, x, p.M, p.K, kBM))) return rc;
    if ((rc = make_map(&mb, w, p.N, p.K, BN / 2))) return rc;
    const int units = ((p.M + 2 * kBM - 1) / (2 * kBM)) * ((p.N + BN - 1) / BN);
    const int pairs = units < pairs_max ? units : pairs_max;
    launch_kernel_clustered(kernel, 2 * pairs, kThreads, smem, 2, stream, ma, mb, p);
    return CITLALI_LAUNCH_CHECK();
}

}  // namespace pair
}  // namespace tc
}  // namespace citlali

using namespace citlali;

// Bytes of x (rows of a band of row tiles, all of K) that should stay in L2 while the weight tiles pass by.
static long g_band_bytes = 32L << 20;

// For tuning: sets the band's size in bytes and returns the one that stood before.
extern "C" long citlali_gemm_tc_pair_set_band_bytes(long bytes) {
    const long before = g_band_bytes;
    if (bytes > 0) g_band_bytes = bytes;
    return before;
}

// The tile width the pair kernel would use for this shape and how many pairs the device runs at once
// (0: it does not run here).
extern "C" int citlali_gemm_tc_pair_plan(int M, int N, int K, int* bn, int* pairs) {
    (void)M; (void)K;
    if (bn) *bn = N >= 256 ? 256 : 128;
    if (pairs) *pairs = N >= 256 ? tc::pair::resident_pairs<256>((size_t)tc::pair::stages_for<256>() * (16384 + 128 * 128) + tc::pair::kEpilogueWarps * tc::kEpilogueStageBytes + 1024)
                                  : tc::pair::resident_pairs<128>((size_t)tc::pair::stages_for<128>() * (16384 + 64 * 128) + tc::pair::kEpilogueWarps * tc::kEpilogueStageBytes + 1024);
    return 0;
}

// y = x . w^T as citlali_gemm_tc computes it (same `mode` bits, same outputs), on pairs of SMs.
// For many rows of x; it takes every M, N and K that citlali_gemm_tc takes.
extern "C" int citlali_gemm_tc_pair(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                                    int mode, int32_t* error_flag, cudaStream_t stream) {
    const bool accumulate = (mode & 1) != 0, swiglu = (mode & 2) != 0;
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0) {
        set_last_error("gemm_tc_pair: the inner size %d must be a positive multiple of 8 (rows of 16-byte multiples for TMA)", K);
        return kBadShape;
    }
    if (((uintptr_t)x | (uintptr_t)w) & 15u) {
        set_last_error("gemm_tc_pair: operands must start on 16-byte boundaries");
        return kBadAlignment;
    }
    if (accumulate && y_dtype != kF32) {
        set_last_error("gemm_tc_pair: accumulation needs a float32 output");
        return kBadDType;
    }
    if (y_dtype != kF32 && y_dtype != kBF16) {
        set_last_error("gemm_tc_pair: output dtype code %d is neither float32 nor bfloat16", y_dtype);
        return kBadDType;
    }
    if (swiglu && (accumulate || y_dtype != kBF16 || N % 32 != 0)) {
        set_last_error("gemm_tc_pair: the gate epilogue needs a bfloat16 output and N a multiple of 32 (N %d)", N);
        return kBadShape;
    }
    tc::pair::Params p;
    p.M = M; p.N = N; p.K = K;
    {
        const long tile_bytes = 2L * tc::pair::kBM * K * 2, tiles_m = (M + 2 * tc::pair::kBM - 1) / (2 * tc::pair::kBM);
        long band = g_band_bytes / tile_bytes;
        if (band < 4) band = 4;
        p.band = (int)(band < tiles_m ? band : tiles_m);
    }
    p.error_flag = error_flag;
    p.out = y;
    p.out_kind = swiglu ? tc::kSwigluBF16 : accumulate ? tc::kAddF32 : (y_dtype == kF32 ? tc::kStoreF32 : tc::kStoreBF16);
    return N >= 256 ? tc::pair::launch<256>(x, w, p, stream) : tc::pair::launch<128>(x, w, p, stream);
}
