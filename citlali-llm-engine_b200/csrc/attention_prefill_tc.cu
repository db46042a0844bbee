// Causal attention of runs of new tokens over the paged cache on the fifth-generation tensor
// cores, for head size 128 and pages of 64 keys.
//
// A block owns an SM and works on TWO query tiles of 128 rows that read the same keys and values:
// two query heads of one key/value group over the same 128 new tokens (when the group has an even
// number of heads), else two consecutive row tiles of one head.  It walks the visible keys 128 at
// a time (two cache pages); each key and value tile is fetched once for both query tiles, which
// halves the traffic from L2, the resource this kernel is otherwise bound by.  Roles:
//   warps 16, 17, one lane each: TMA producers of the key and of the value tiles (128-byte swizzle; a
//                     tile is two 64-wide halves of the head), two tiles deep.
//   warp 18, one lane: MMA issuer for both query tiles.  S = Q K^T (tcgen05.mma, both operands
//                     K-major in shared memory) into tensor memory; O += P V with P read from tensor
//                     memory (it lies over the scores it came from) and V, as stored (head dimension
//                     contiguous), as an MN-major shared-memory operand.  The scores of a query
//                     tile's next key tile are issued right after its P V, so one query tile's
//                     softmax runs while the other's MMAs do.  An MMA of 128 x 128 x 16 keeps the
//                     tensor pipe busy for 64 clocks and the pipe takes only a few MMAs ahead, while
//                     a look at an mbarrier costs this thread 100 to 180 clocks even when the barrier
//                     has long been passed (measured): so every barrier is looked at BEFORE the MMAs
//                     of the group ahead of the one that needs it are issued, the answer is used
//                     after them, and a key tile's keys and values share one barrier each way.
//   warps 0-7, 8-15:  softmax of query tile 0 and 1.  Two threads own one query row: the warps of a
//                     32-row quarter take the tile's keys 0-63 and 64-127 (a scheduler then has two
//                     warps of a tile to switch between: one alone waits on latencies, not on the
//                     special-function unit).  Exponentials are taken against the reference the row
//                     already has, without a maximum: the reference only has to keep P and the sums in
//                     range, and the tile's sum tells whether it did.  If it did not for either half
//                     (or the row has no reference yet: the first tile), both warps take a second pass
//                     with the row's true maximum and rescale their columns of O.  Each half keeps its
//                     own sum against the common reference, so the result is exact.  The two warps
//                     meet on an mbarrier of their own (votes, maxima and sums go through shared
//                     memory).  Each half stores its P over its own scores: keys 0-63 in columns 0-31,
//                     keys 64-127 in columns 64-95.  At the end each thread divides its half row of O
//                     by the row's sum and stores it.
// Tensor memory: 512 columns, per query tile 128 of scores / P and 128 of output.  Shared memory:
// two query tiles, two key tiles, two value tiles of 32 KB.
//
// Formulas: the reference's (attention_scores_kernel / attention_values_kernel,
// src/compute/cuda/kernels.cu:545-649): s = q.k / sqrt(d), keys lo..p for the token at position
// p, query head j reads key/value head j / (heads / kv_heads); softmax and sums in float.
// Every mbarrier wait is bounded and reports through the error word.
#include "api.h"
#include "common.cuh"
#include "tc_common.cuh"
#include "tc_host.h"

namespace citlali {
namespace fatc {

using namespace tc;

constexpr int kD = 128, kTileQ = 128, kTileK = 128, kPage = 64;
constexpr int kWarpLoadK = 16, kWarpLoadV = 17, kWarpMma = 18;
constexpr int kThreads = 608;
constexpr int kHalfKeys = kTileK / 2;                  // keys of a tile that one softmax thread works on
constexpr uint32_t kHalfTile = 128 * 128;              // bytes of [128 rows x 64 bfloat16]
constexpr uint32_t kTileBytes = 2 * kHalfTile;         // [128 x 128] bfloat16
// tensor memory columns of query tile b: kSubCols * b + ...; P overwrites the scores it came from: the P of
// keys 64 h .. 64 h + 63 (32 columns of two bfloat16) lies at the start of those keys' own 64 score columns
constexpr uint32_t kSubCols = 256, kColS = 0, kColP = 0, kColO = 128, kTmemCols = 512;

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
// Waits for this thread's tensor-memory loads; the 32 registers go through the statement so that
// nothing that uses them is scheduled before it.
__device__ __forceinline__ void tmem_ld_wait32(uint32_t* r) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
        : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
          "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
          "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
          "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
        :: "memory");
}
// The same for 16 registers of tmem_ld16.
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
        : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
          "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
        :: "memory");
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

// A look at an mbarrier costs the issuing thread 100 to 180 clocks during which it issues nothing, and the tensor
// pipe, which takes only a few MMAs ahead, runs dry.  In these two the look (`mbarrier.try_wait`, one try) is
// issued FIRST and its answer is taken LAST, with a group's eight MMAs between them in one statement, so that the
// MMAs go out while the look is on its way.  Returns whether phase `parity` of `bar` had completed.
//
// S[128 x 128] = A . B^T over the head size 128: eight K slices; an operand's two 64-element halves lie
// `half_units` (in 16-byte units) apart, a slice within a half 32 bytes (2 units) after the one before.
__device__ __forceinline__ bool mma_scores_and_look(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                    uint32_t bar, uint32_t parity) {
    uint32_t seen;
    asm volatile(
        "{\n"
        ".reg .pred look, yes, no;\n"
        ".reg .b64 a, b;\n"
        "setp.eq.u32 yes, 0, 0;\n"
        "setp.ne.u32 no, 0, 0;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 look, [%5], %6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %4, no;\n"
        "add.u64 a, %2, 2;\n add.u64 b, %3, 2;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %4, yes;\n"
        "add.u64 a, %2, 4;\n add.u64 b, %3, 4;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %4, yes;\n"
        "add.u64 a, %2, 6;\n add.u64 b, %3, 6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %4, yes;\n"
        "add.u64 a, %2, 1024;\n add.u64 b, %3, 1024;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %4, yes;\n"
        "add.u64 a, %2, 1026;\n add.u64 b, %3, 1026;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %4, yes;\n"
        "add.u64 a, %2, 1028;\n add.u64 b, %3, 1028;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %4, yes;\n"
        "add.u64 a, %2, 1030;\n add.u64 b, %3, 1030;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a, b, %4, yes;\n"
        "selp.b32 %0, 1, 0, look;\n"
        "}"
        : "=r"(seen) : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(bar), "r"(parity) : "memory");
    return seen != 0;
}
// O[128 x 128] (+)= P . V over a tile's 128 keys: eight slices of 16 keys; P's slice j lies at tensor-memory column
// (j / 4) * 64 + (j % 4) * 8 of `tmem_p` (each half of the keys has its P at the start of its own scores), V's
// slice is 16 rows of 128 bytes (128 units) after the one before.  `accumulate` = 0 starts O anew.
__device__ __forceinline__ bool mma_values_and_look(uint32_t tmem_d, uint32_t tmem_p, uint64_t desc_v, uint32_t idesc,
                                                    uint32_t accumulate, uint32_t bar, uint32_t parity) {
    uint32_t seen;
    asm volatile(
        "{\n"
        ".reg .pred look, yes, first;\n"
        ".reg .b64 v;\n"
        ".reg .b32 pp;\n"
        "setp.eq.u32 yes, 0, 0;\n"
        "setp.ne.b32 first, %5, 0;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 look, [%6], %7;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], [%2], %3, %4, first;\n"
        "add.u32 pp, %2, 8;\n add.u64 v, %3, 128;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], [pp], v, %4, yes;\n"
        "add.u32 pp, %2, 16;\n add.u64 v, %3, 256;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], [pp], v, %4, yes;\n"
        "add.u32 pp, %2, 24;\n add.u64 v, %3, 384;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], [pp], v, %4, yes;\n"
        "add.u32 pp, %2, 64;\n add.u64 v, %3, 512;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], [pp], v, %4, yes;\n"
        "add.u32 pp, %2, 72;\n add.u64 v, %3, 640;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], [pp], v, %4, yes;\n"
        "add.u32 pp, %2, 80;\n add.u64 v, %3, 768;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], [pp], v, %4, yes;\n"
        "add.u32 pp, %2, 88;\n add.u64 v, %3, 896;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], [pp], v, %4, yes;\n"
        "selp.b32 %0, 1, 0, look;\n"
        "}"
        : "=r"(seen) : "r"(tmem_d), "r"(tmem_p), "l"(desc_v), "r"(idesc), "r"(accumulate), "r"(bar), "r"(parity) : "memory");
    return seen != 0;
}
static_assert(kHalfTile >> 4 == 1024 && kHalfKeys == 64 && kD == 128 && kTileK == 128,
              "the offsets written into mma_scores_and_look and mma_values_and_look are those of 128 x 128 tiles");

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
    int pair_heads;                      // 1: the two query tiles are heads 2x, 2x+1; 0: row tiles 2y, 2y+1 of head x
    float scale_log2;
    int32_t* error_flag;
};

// One of the block's two query tiles: its head, its first row within the sequence's new tokens, and the
// key tiles it reads (none when it has no rows).
struct QueryTile {
    int head, q0, tile_lo, tile_hi;
    __device__ bool reads(int t) const { return t >= tile_lo && t <= tile_hi; }
};

__global__ void __launch_bounds__(kThreads, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, Params p) {
    extern __shared__ uint8_t smem_raw[];
    // kv_full[stage]: the keys and the values of a tile have landed (both producers arrive with their bytes);
    // kv_empty[stage]: the MMAs on them have finished
    __shared__ __align__(8) uint64_t q_bar, kv_full[2], kv_empty[2], s_full[2], p_full[2], o_done[2];
    __shared__ __align__(8) uint64_t pair_bar[2][4];         // the two softmax warps of (query tile, quarter) meet here
    __shared__ float pair_value[2][2][kTileQ];               // [query tile][half][row]: this half's maximum, for the other half
    __shared__ float pair_sum[2][2][kTileQ];                 // the same for the sums at the end (a thread that is done with its
                                                             // last tile must not write over a maximum its partner has yet to read)
    __shared__ int pair_vote[2][4][2];                       // [query tile][quarter][half]: this half wants the second pass
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t s_q = base, s_k = base + 2 * kTileBytes, s_v = base + 4 * kTileBytes;      // two tiles each
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
        abort_word = 0;
        mbar_init(smem_u32(&q_bar), 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&kv_full[i]), 2);
            mbar_init(smem_u32(&kv_empty[i]), 1);
            mbar_init(smem_u32(&s_full[i]), 1);
            mbar_init(smem_u32(&p_full[i]), 8);
            mbar_init(smem_u32(&o_done[i]), 1);
            for (int qd = 0; qd < 4; ++qd) mbar_init(smem_u32(&pair_bar[i][qd]), 2);
        }
        fence_barrier_init();
        fence_async_proxy();
    }
    if (warp == kWarpMma) {
        tmem_alloc(smem_u32(&tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    dependents_may_launch();                                 // only now: this block holds its tensor memory

    wait_for_predecessor();                                  // everything below reads what earlier kernels wrote
    // blocks are handed out x fastest: all heads of the last rows (the ones that see the most keys)
    // first, then all heads of the rows before them, and so on
    const int seq = blockIdx.z;
    const int row0 = p.seq_start[seq], n_new = p.seq_start[seq + 1] - row0;
    const int past = p.seq_past[seq];
    const int y = gridDim.y - 1 - blockIdx.y;
    QueryTile qt[2];
    int t_lo = INT_MAX, t_hi = -1, last_key = -1;            // the block's key tiles and its last visible key
#pragma unroll
    for (int b = 0; b < 2; ++b) {
        qt[b].head = p.pair_heads ? 2 * blockIdx.x + b : blockIdx.x;
        qt[b].q0 = (p.pair_heads ? y : 2 * y + b) * kTileQ;
        if (qt[b].q0 < n_new) {
            const int first_pos = past + qt[b].q0, last_pos = past + min(qt[b].q0 + kTileQ, n_new) - 1;
            const int lo_key = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
            qt[b].tile_lo = lo_key / kTileK; qt[b].tile_hi = last_pos / kTileK;
            t_lo = min(t_lo, qt[b].tile_lo); t_hi = max(t_hi, qt[b].tile_hi); last_key = max(last_key, last_pos);
        } else {
            qt[b].tile_lo = 0; qt[b].tile_hi = -1;
        }
    }
    const int g = qt[0].head / (p.nq / p.nkv);               // both query tiles read this key/value head
    const int32_t* pages = p.page_table + (size_t)p.seq_slot[seq] * p.page_table_stride;

    if (warp == kWarpLoadK || warp == kWarpLoadV) {
        if (lane == 0 && t_hi >= t_lo) {
            const bool is_k = warp == kWarpLoadK;
            if (is_k) {
                // rows past the end of q read as zeros; a query tile without rows is loaded and never used
                mbar_arrive_expect_tx(smem_u32(&q_bar), 2 * kTileBytes);
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    tma_load_2d(s_q + b * kTileBytes, &map_q, qt[b].head * kD, row0 + qt[b].q0, smem_u32(&q_bar));
                    tma_load_2d(s_q + b * kTileBytes + kHalfTile, &map_q, qt[b].head * kD + 64, row0 + qt[b].q0, smem_u32(&q_bar));
                }
            }
            const CUtensorMap* map = is_k ? &map_k : &map_v;
            for (int t = t_lo; t <= t_hi; ++t) {
                const int i = t - t_lo, st = i & 1;
                const int key0 = t * kTileK;
                // two pages per tile; a page that lies wholly past the last visible key is not fetched (the
                // first page stands in): its scores are masked and its values are multiplied by zeros
                const int page_a = pages[key0 / kPage];
                const bool second = key0 + kPage <= last_key;
                const int page_b = second ? pages[key0 / kPage + 1] : page_a;
                const int ra = (page_a * p.nkv + g) * kPage, rb = (page_b * p.nkv + g) * kPage;
                const uint32_t full = smem_u32(&kv_full[st]), empty = smem_u32(&kv_empty[st]);
                const uint32_t dst = (is_k ? s_k : s_v) + st * kTileBytes;
                if (!mbar_wait(empty, ((i >> 1) & 1u) ^ 1u, abort_flag, p.error_flag, is_k ? 201 : 210)) break;
                mbar_arrive_expect_tx(full, kTileBytes);
                tma_load_2d(dst, map, 0, ra, full);
                tma_load_2d(dst + 64 * 128, map, 0, rb, full);
                tma_load_2d(dst + kHalfTile, map, 64, ra, full);
                tma_load_2d(dst + kHalfTile + 64 * 128, map, 64, rb, full);
            }
        }
        __syncwarp();
    } else if (warp == kWarpMma) {
        if (lane == 0 && t_hi >= t_lo) {
            constexpr uint32_t idesc_qk = instr_desc_bf16(kTileQ, kTileK);
            constexpr uint32_t idesc_pv = instr_desc_bf16(kTileQ, kD) | (1u << 16);        // B is MN-major
            bool ok = true;
            // Every descriptor is made once, before the loop; a K slice is an addition of a constant to its address
            // field (16-byte units; the tiles are far below the field's 256 KB).
            constexpr uint64_t kTileUnits = kTileBytes >> 4;     // the second tile of a pair, in the address field's units
            const uint64_t dq0 = smem_desc_sw128(s_q, 0), dk0 = smem_desc_sw128(s_k, 0), dv0 = smem_desc_mn_sw128(s_v, kHalfTile);
            // A barrier this thread will need: looked at once ahead of time (`seen`), waited for only if that look
            // came too early.
            auto look_kv = [&](int t) -> bool {
                return mbar_try_wait(smem_u32(&kv_full[(t - t_lo) & 1]), ((t - t_lo) >> 1) & 1u);
            };
            auto need_kv = [&](int t, bool seen) -> bool {
                if (!seen && !mbar_wait(smem_u32(&kv_full[(t - t_lo) & 1]), ((t - t_lo) >> 1) & 1u, abort_flag, p.error_flag, 203)) return false;
                return true;
            };
            auto need_p = [&](int b, int t, bool seen) -> bool {
                if (!seen && !mbar_wait(smem_u32(&p_full[b]), (uint32_t)(t - qt[b].tile_lo) & 1u, abort_flag, p.error_flag, 205)) return false;
                tc_fence_after();
                return true;
            };
            // MMAs of one thread run and finish in the order they are issued: the scores of tile t+1, issued after
            // P V of tile t, overwrite P only when that product has read it, and their commit also says that P V of
            // tile t has finished (the softmax threads rely on it when they rescale O).
            // Each group of eight MMAs carries a look at the barrier that the NEXT group will need (see
            // mma_scores_and_look); `look_bar` 0 means there is nothing to look at (the Q barrier, long passed, stands in).
            const uint32_t passed_bar = smem_u32(&q_bar);
            auto issue_qk = [&](int b, int t, uint32_t look_bar, uint32_t look_parity) -> bool {
                const uint64_t a0 = dq0 + (b ? kTileUnits : 0), b0 = dk0 + (((t - t_lo) & 1) ? kTileUnits : 0);
                const bool seen = mma_scores_and_look(tmem + b * kSubCols + kColS, a0, b0, idesc_qk,
                                                      look_bar ? look_bar : passed_bar, look_bar ? look_parity : 0u);
                mma_commit(smem_u32(&s_full[b]));
                return seen && look_bar != 0;
            };
            auto issue_pv = [&](int b, int t, uint32_t look_bar, uint32_t look_parity) -> bool {
                const uint64_t v0 = dv0 + (((t - t_lo) & 1) ? kTileUnits : 0);
                const bool seen = mma_values_and_look(tmem + b * kSubCols + kColO, tmem + b * kSubCols + kColP, v0, idesc_pv,
                                                      t > qt[b].tile_lo ? 1u : 0u, look_bar ? look_bar : passed_bar,
                                                      look_bar ? look_parity : 0u);
                if (t == qt[b].tile_hi) mma_commit(smem_u32(&o_done[b]));
                return seen && look_bar != 0;
            };
            auto kv_bar = [&](int t) -> uint32_t { return smem_u32(&kv_full[(t - t_lo) & 1]); };
            auto kv_parity = [&](int t) -> uint32_t { return ((t - t_lo) >> 1) & 1u; };
            auto p_parity = [&](int b, int t) -> uint32_t { return (uint32_t)(t - qt[b].tile_lo) & 1u; };
            ok = mbar_wait(smem_u32(&q_bar), 0, abort_flag, p.error_flag, 202) && need_kv(t_lo, false);
            if (ok) {
                tc_fence_after();
                if (qt[0].reads(t_lo)) issue_qk(0, t_lo, 0, 0);
                if (qt[1].reads(t_lo)) issue_qk(1, t_lo, 0, 0);
            }
            // the order of a key tile's groups of MMAs: P V of query tile 0 (looking at the next tile's keys and
            // values), its next scores (looking at P of query tile 1), P V of query tile 1, the next scores of query
            // tile 1 (looking at the next P of query tile 0, most likely too early: then it is waited for)
            bool seen_p0 = false;                             // P of query tile 0 for tile t
            for (int t = t_lo; t <= t_hi && ok; ++t) {
                const bool more = t + 1 <= t_hi;
                bool seen_kv = false, seen_p1 = false;
                if (qt[0].reads(t)) {
                    if (!need_p(0, t, seen_p0)) { ok = false; break; }
                    seen_kv = issue_pv(0, t, more ? kv_bar(t + 1) : 0u, more ? kv_parity(t + 1) : 0u);
                } else if (more) {
                    seen_kv = look_kv(t + 1);
                }
                if (more) {
                    if (!need_kv(t + 1, seen_kv)) { ok = false; break; }
                    if (qt[0].reads(t + 1)) {
                        tc_fence_after();
                        seen_p1 = issue_qk(0, t + 1, qt[1].reads(t) ? smem_u32(&p_full[1]) : 0u, qt[1].reads(t) ? p_parity(1, t) : 0u);
                    }
                }
                if (qt[1].reads(t)) {
                    if (!need_p(1, t, seen_p1)) { ok = false; break; }
                    issue_pv(1, t, 0, 0);
                }
                // the tile's keys and values are free when everything issued so far has finished
                mma_commit(smem_u32(&kv_empty[(t - t_lo) & 1]));
                seen_p0 = false;
                if (more && qt[1].reads(t + 1)) {
                    const bool look = qt[0].reads(t + 1);
                    seen_p0 = issue_qk(1, t + 1, look ? smem_u32(&p_full[0]) : 0u, look ? p_parity(0, t + 1) : 0u);
                }
            }
        }
        __syncwarp();
    } else {
        // softmax of query tile b: this thread owns keys 64 half .. 64 half + 63 of its row `r`
        const int b = warp >> 3, half = (warp >> 2) & 1, quarter = warp & 3;
        const QueryTile me = b ? qt[1] : qt[0];
        const int tiles = me.tile_hi - me.tile_lo + 1;        // 0 for a query tile without rows
        const int r = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const uint32_t sub = tmem + b * kSubCols + lane_addr;
        const uint32_t s_addr = sub + kColS + half * kHalfKeys;       // this thread's 64 scores; its P goes over their start
        const int pos = past + me.q0 + r;
        const int lo = p.window > 0 ? pos - p.window + 1 : 0;
        const int warp_pos = past + me.q0 + quarter * 32;
        const uint32_t meet = smem_u32(&pair_bar[b][quarter]);
        uint32_t meetings = 0;
        float m_ref = -INFINITY, l = 0.0f;                    // the row's reference maximum (raw score units), this half's sum
        bool ok = true;
        // Both warps of the pair arrive and wait; what either wrote to shared memory before is visible to both after.
        auto meet_partner = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(meet);
            const bool met = mbar_wait(meet, meetings & 1u, abort_flag, p.error_flag, 211);
            ++meetings;
            return met;
        };
        for (int t = 0; t < tiles && ok; ++t) {
            const int key0 = (me.tile_lo + t) * kTileK + half * kHalfKeys;
            if (!mbar_wait(smem_u32(&s_full[b]), t & 1u, abort_flag, p.error_flag, 207)) { ok = false; break; }
            tc_fence_after();
            const bool masked = key0 + kHalfKeys - 1 > warp_pos || (p.window > 0 && key0 < warp_pos + 31 - p.window + 1);
            uint32_t pk[32];                                  // P of this half row, two bfloat16 a register
            uint32_t a[16], bb[16];
            auto mask16 = [&](uint32_t (&h)[16], int c_base) {
                if (masked) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int key = key0 + c_base + c;
                        if (key > pos || key < lo) h[c] = 0xff800000u;                    // -inf
                    }
                }
            };
            bool two_pass = t == 0;
            if (!two_pass) {
                // One pass, 16 scores at a time while the next 16 are on their way from tensor memory.  A P above
                // 2^15 makes the sum exceed 2^15, and a sum above 2^15 needs a P above 2^8: past that the
                // reference is renewed.  The scores stay in tensor memory until P is stored over them.
                const float ref = m_ref == -INFINITY ? 0.0f : m_ref * p.scale_log2;
                float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
                auto chunk = [&](uint32_t (&h)[16], int c_base) {
                    mask16(h, c_base);
#pragma unroll
                    for (int c = 0; c < 16; c += 8) {
                        float e[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) e[i] = ex2(fmaf(__uint_as_float(h[c + i]), p.scale_log2, -ref));
                        s0 += e[0] + e[1]; s1 += e[2] + e[3]; s2 += e[4] + e[5]; s3 += e[6] + e[7];
#pragma unroll
                        for (int i = 0; i < 8; i += 2) {
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(e[i], e[i + 1]);
                            pk[(c_base + c + i) >> 1] = *reinterpret_cast<uint32_t*>(&h2);
                        }
                    }
                };
                tmem_ld16(s_addr, a);
                tmem_ld_wait16(a);
                tmem_ld16(s_addr + 16, bb);
                chunk(a, 0);
                tmem_ld_wait16(bb);
                tmem_ld16(s_addr + 32, a);
                chunk(bb, 16);
                tmem_ld_wait16(a);
                tmem_ld16(s_addr + 48, bb);
                chunk(a, 32);
                tmem_ld_wait16(bb);
                chunk(bb, 48);
                const float tile_sum = (s0 + s1) + (s2 + s3);
                const bool in_range = tile_sum <= 32768.0f && m_ref != -INFINITY;      // false for inf and NaN too
                const bool mine = __any_sync(0xffffffffu, !in_range);
                if (lane == 0) pair_vote[b][quarter][half] = mine ? 1 : 0;
                if (!meet_partner()) { ok = false; break; }
                two_pass = mine || pair_vote[b][quarter][half ^ 1] != 0;
                if (!two_pass) l += tile_sum;
            }
            if (two_pass) {
                // The row's maximum first (this half's, then the other's through shared memory), then the exponentials
                // against a reference that grows only when the maximum has run away from it by more than 2^8.
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll 1
                for (int c_base = 0; c_base < kHalfKeys; c_base += 16) {
                    tmem_ld16(s_addr + c_base, a);
                    tmem_ld_wait16(a);
                    mask16(a, c_base);
#pragma unroll
                    for (int c = 0; c < 16; c += 2) { mx0 = fmaxf(mx0, __uint_as_float(a[c])); mx1 = fmaxf(mx1, __uint_as_float(a[c + 1])); }
                }
                pair_value[b][half][r] = fmaxf(mx0, mx1);
                if (!meet_partner()) { ok = false; break; }
                const float mx = fmaxf(fmaxf(mx0, mx1), pair_value[b][half ^ 1][r]);
                // (this slot is written again only after the partner has read it: the next tile's scores, which both wait
                // for, are issued after the partner's arrival on p_full, which follows its read)
                float alpha = 1.0f;
                const bool grow = (mx - m_ref) * p.scale_log2 > 8.0f || m_ref == -INFINITY;
                if (grow && mx > -INFINITY) {
                    alpha = m_ref == -INFINITY ? 0.0f : ex2((m_ref - mx) * p.scale_log2);
                    m_ref = mx;
                    l *= alpha;
                }
                const bool rescale = t > 0 && __any_sync(0xffffffffu, alpha != 1.0f);
                const float ref = m_ref == -INFINITY ? 0.0f : m_ref * p.scale_log2;
                float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll 1
                for (int c_base = 0; c_base < kHalfKeys; c_base += 16) {
                    tmem_ld16(s_addr + c_base, a);
                    tmem_ld_wait16(a);
                    mask16(a, c_base);
#pragma unroll
                    for (int c = 0; c < 16; c += 4) {
                        const float e0 = ex2(fmaf(__uint_as_float(a[c]), p.scale_log2, -ref));
                        const float e1 = ex2(fmaf(__uint_as_float(a[c + 1]), p.scale_log2, -ref));
                        const float e2 = ex2(fmaf(__uint_as_float(a[c + 2]), p.scale_log2, -ref));
                        const float e3 = ex2(fmaf(__uint_as_float(a[c + 3]), p.scale_log2, -ref));
                        sum0 += e0 + e1; sum1 += e2 + e3;
                        __nv_bfloat162 h01 = __floats2bfloat162_rn(e0, e1), h23 = __floats2bfloat162_rn(e2, e3);
                        // a loop that is not unrolled cannot index registers: the chunk's P goes to tensor memory at the end
                        bb[c >> 1] = *reinterpret_cast<uint32_t*>(&h01);
                        bb[(c >> 1) + 1] = *reinterpret_cast<uint32_t*>(&h23);
                    }
                    // this chunk's P (8 registers) over the start of the scores already read: chunk i's P lies in
                    // columns 8 i .. 8 i + 7, behind the 16 i .. 16 i + 15 its scores came from and never ahead of a
                    // chunk still to be read
                    uint32_t w8[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) w8[i] = bb[i];
                    tmem_st8(s_addr + (c_base >> 1), w8);
                }
                l += sum0 + sum1;
                // O is quiet when it is rescaled: this tile's scores were issued after P V of the tile before by the same
                // thread, MMAs finish in order, and the scores' arrival was waited for above
                if (rescale) {
#pragma unroll 1
                    for (int c0 = 0; c0 < kHalfKeys; c0 += 16) {
                        tmem_ld16(sub + kColO + half * kHalfKeys + c0, a);
                        tmem_ld_wait16(a);
#pragma unroll
                        for (int c = 0; c < 16; ++c) a[c] = __float_as_uint(__uint_as_float(a[c]) * alpha);
                        tmem_st16(sub + kColO + half * kHalfKeys + c0, a);
                    }
                }
            } else {
                tmem_st32(s_addr, pk);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[b]));
        }
        // the row's sum is the two halves' sums; each thread normalises and stores its 64 columns of O
        if (ok && tiles > 0) {
            pair_sum[b][half][r] = l;
            ok = meet_partner();
            l += pair_sum[b][half ^ 1][r];
        }
        if (ok && tiles > 0 && mbar_wait(smem_u32(&o_done[b]), 0, abort_flag, p.error_flag, 209)) {
            tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const bool store = me.q0 + r < n_new;
            __nv_bfloat16* dst = p.out + (size_t)(row0 + me.q0 + r) * p.out_stride + (size_t)me.head * kD + half * kHalfKeys;
#pragma unroll 1
            for (int c0 = 0; c0 < kHalfKeys; c0 += 16) {
                uint32_t ov[16];
                tmem_ld16(sub + kColO + half * kHalfKeys + c0, ov);
                tmem_ld_wait16(ov);
                if (store) {
#pragma unroll
                    for (int c = 0; c < 16; c += 8) {
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
    if (warp == kWarpMma) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// [rows, row_elems] bfloat16, row pitch `pitch_elems`, as boxes of [box_rows, 64] with 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_elems, uint64_t pitch_elems, int box_rows) {
    return tc::make_bf16_map(map, base, rows, row_elems, pitch_elems, box_rows, "attention_prefill_tc");
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
    // two heads of a key/value group share a block when groups have an even number of heads, else two row tiles
    p.pair_heads = (nq / nkv) % 2 == 0 ? 1 : 0;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.error_flag = error_flag;
    const size_t smem = (size_t)6 * fatc::kTileBytes + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(fatc::attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int row_tiles = (max_new + fatc::kTileQ - 1) / fatc::kTileQ;
    dim3 grid(p.pair_heads ? nq / 2 : nq, p.pair_heads ? row_tiles : (row_tiles + 1) / 2, sequences);
    launch_kernel(fatc::attention_prefill_tc_kernel, grid, fatc::kThreads, smem, stream, mq, mk, mv, p);
    return CITLALI_LAUNCH_CHECK();
}
