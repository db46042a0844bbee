// Inline PTX for the Blackwell tensor-core path: mbarriers, TMA tile loads, tcgen05 MMA with
// accumulators in tensor memory, and waits that give up after a time limit instead of hanging.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace citlali {
namespace tc {

constexpr uint64_t kWaitLimitNs = 2000000000ull;   // a wait that lasts 2 s has failed

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t global_timer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_async_proxy() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Wait for a phase of an mbarrier, but not for ever: returns false when another thread of the
// block has given up (`*abort_flag`), or after kWaitLimitNs, in which case it records `code`
// in error_flag[1] (and the block in error_flag[2]) and raises the block's abort flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int32_t* error_flag, int code, uint64_t limit_ns = kWaitLimitNs) {
    uint64_t start = 0;
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 31u) == 0u) {
            if (*abort_flag) return false;
            if (start == 0) start = global_timer();         // the clock is read only once the wait is long
            if (global_timer() - start > limit_ns) {
                *abort_flag = 1;
                if (error_flag) {
                    atomicExch(error_flag + 1, code);
                    atomicExch(error_flag + 2, (int)blockIdx.x);
                }
                return false;
            }
            __nanosleep(64);
        }
    }
}

// Brings a tensor map (a kernel parameter) into the descriptor cache ahead of its first use.
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// One 2-D tile [box rows x box cols] from a row-major matrix into shared memory; completion
// is counted in bytes on `bar`.  `c_inner` (elements along the row) must make a 16-byte
// multiple; here it is always a multiple of 64 bfloat16.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c_inner, int c_outer, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c_inner), "r"(c_outer), "r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] . B[smem]^T, bfloat16 operands, float accumulators, one CTA.
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// When every MMA issued so far by this thread has finished, arrive once on `bar`.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 16 consecutive accumulator columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor: K-major tile whose rows are 128 bytes (64 bfloat16),
// 128-byte swizzle, groups of 8 rows 1024 bytes apart; the tile starts on a 1024-byte boundary
// and `byte_offset` (a multiple of 32 below 128) selects the 16-element K slice.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t tile_addr, uint32_t byte_offset) {
    uint64_t d = 0;
    d |= (uint64_t)(((tile_addr + byte_offset) >> 4) & 0x3FFFu);     // start address
    d |= (uint64_t)1 << 16;                                         // leading byte offset (unused here)
    d |= (uint64_t)(1024 >> 4) << 32;                               // stride byte offset
    d |= (uint64_t)1 << 46;                                         // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                                         // 128-byte swizzle
    return d;
}

// Instruction descriptor: bfloat16 x bfloat16 -> float, both operands K-major, M x N tile.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- two blocks of a cluster on one MMA (cta_group::2) ---------------------------------------
// The block with cluster rank 0 issues the MMAs; each block supplies its half of the operands from
// its own shared memory and holds its 128 rows of the accumulator in its own tensor memory.

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The shared-memory address `addr` of this block, as the block with rank `rank` of the cluster has it.
__device__ __forceinline__ uint32_t cluster_addr(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on an mbarrier of another block of the cluster (`bar` from cluster_addr).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// A tile into this block's shared memory whose bytes are counted on an mbarrier of either block of the
// pair (`bar` is a shared::cluster address).  No multicast: the tile goes to this block alone.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c_inner, int c_outer, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c_inner), "r"(c_outer), "r"(bar) : "memory");
}
// Tensor memory for the pair: the same warp of both blocks executes each of these.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// D[tmem of both blocks, 256 rows] (+)= A . B^T: A's rows 128 r .. and B's rows (N/2) r .. come from
// the shared memory of the block with rank r, at the same addresses in both.
__device__ __forceinline__ void mma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// When every MMA issued so far by this thread has finished, arrive once on the mbarrier at `bar`'s
// address in every block of the cluster whose rank is set in `mask`.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}

// ---- epilogue: a warp's 32 rows x 16 values, written with full sectors ------------------------
// A thread holds 16 consecutive outputs of ITS row (lane = row), so a plain store touches 32 rows with 16
// bytes each.  Here the warp turns the values round in a private shared-memory area of kEpilogueStageBytes
// and writes them so that every instruction covers whole 32-byte sectors: 8 rows x 64 bytes (float) or
// 16 rows x 32 bytes (bfloat16).  `out` points at row `row0`, column j0 of the output; rows from `rows_left`
// on do not exist.
constexpr uint32_t kEpilogueStageBytes = 32 * 20 * 4;

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
// The outputs stream out once: they are marked to leave L2 first, so that they do not push out the
// operand tiles that other blocks are about to read again.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void red_add_v4(float* addr, uint4 v, uint64_t policy) {
    asm volatile("red.global.add.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;"
                 ::"l"(addr), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)), "l"(policy) : "memory");
}
__device__ __forceinline__ void st_global_v4_hint(void* addr, uint4 v, uint64_t policy) {
    asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;"
                 ::"l"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(policy) : "memory");
}
// 16 floats a row: stored, or added to what is there (one add per element, by one thread: the same sum
// as a load, an add and a store).
__device__ __forceinline__ void warp_rows_out_f32(uint32_t stage, const float (&v)[16], float* out, size_t pitch, int rows_left,
                                                  int lane, bool add, uint64_t policy) {
#pragma unroll
    for (int k = 0; k < 4; ++k)
        st_shared_v4(stage + (uint32_t)(lane * 20 + 4 * k) * 4u, __float_as_uint(v[4 * k]), __float_as_uint(v[4 * k + 1]),
                     __float_as_uint(v[4 * k + 2]), __float_as_uint(v[4 * k + 3]));
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int r = it * 8 + (lane >> 2), cw = (lane & 3) * 4;
        const uint4 t = ld_shared_v4(stage + (uint32_t)(r * 20 + cw) * 4u);
        if (r < rows_left) {
            float* dst = out + (size_t)r * pitch + cw;
            if (add) red_add_v4(dst, t, policy); else st_global_v4_hint(dst, t, policy);
        }
    }
    __syncwarp();
}
// 16 bfloat16 a row, given as 8 words of two.
__device__ __forceinline__ void warp_rows_out_bf16(uint32_t stage, const uint32_t (&w)[8], __nv_bfloat16* out, size_t pitch, int rows_left,
                                                   int lane, uint64_t policy) {
#pragma unroll
    for (int k = 0; k < 2; ++k)
        st_shared_v4(stage + (uint32_t)(lane * 12 + 4 * k) * 4u, w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int r = it * 16 + (lane >> 1), cw = (lane & 1) * 4;
        const uint4 t = ld_shared_v4(stage + (uint32_t)(r * 12 + cw) * 4u);
        if (r < rows_left) st_global_v4_hint(out + (size_t)r * pitch + cw * 2, t, policy);
    }
    __syncwarp();
}

// ---- what a product kernel's epilogue does with its values (rows of x on the tensor memory's lanes) ----------

enum OutKind : int { kStoreBF16 = 0, kStoreF32 = 1, kAddF32 = 2, kSwigluBF16 = 4 };

// silu(g) * u with the fast exponential and the approximate division (a few ulp, before rounding to bfloat16)
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// 16 finished values of row i of x, output features j0 .. j0+15 (c0 = j0 within the tile), of a product
// y[M, N]: stored as bfloat16 or float32, added to float32, or, under the gate epilogue, kept (a gate run, even
// chunks) and then combined with the up run that follows into y[M, N/2] = silu(gate) * up.  Whole chunks of
// whole 32-row groups leave through the warp's area at `epilogue_stage` so that every store covers whole sectors.
__device__ __forceinline__ void finish_rows(const float (&v)[16], int i, int j0, int c0, float (&gate_keep)[16], void* out,
                                            int out_kind, int M, int N, uint32_t epilogue_stage, int lane, uint64_t out_policy) {
    float* outf = (float*)out;
    __nv_bfloat16* outh = (__nv_bfloat16*)out;
    if (out_kind == kSwigluBF16) {
        // Weight rows alternate in runs of 16: gate rows, then the up rows of the same outputs.
        const int half_n = N >> 1;
        if ((c0 & 16) == 0) {
#pragma unroll
            for (int c = 0; c < 16; ++c) gate_keep[c] = v[c];
        } else if (j0 + 16 <= N && (half_n % 8) == 0) {
            uint32_t w[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                __nv_bfloat162 h2 = __floats2bfloat162_rn(silu_mul(gate_keep[2 * c], v[2 * c]),
                                                          silu_mul(gate_keep[2 * c + 1], v[2 * c + 1]));
                w[c] = *reinterpret_cast<uint32_t*>(&h2);
            }
            const int row0 = i - lane;
            warp_rows_out_bf16(epilogue_stage, w, outh + (size_t)row0 * half_n + ((j0 - 16) >> 1), (size_t)half_n, M - row0, lane, out_policy);
        } else if (i < M && j0 - 16 < N) {
            const size_t o = (size_t)i * half_n + ((j0 - 16) >> 1);
            if (j0 + 16 <= N && (half_n % 8) == 0) {
                uint32_t w[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(silu_mul(gate_keep[2 * c], v[2 * c]),
                                                              silu_mul(gate_keep[2 * c + 1], v[2 * c + 1]));
                    w[c] = *reinterpret_cast<uint32_t*>(&h2);
                }
                uint4* dst = reinterpret_cast<uint4*>(outh + o);
                dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
#pragma unroll
                for (int c = 0; c < 16; ++c)
                    if (((j0 - 16) >> 1) + c < half_n) outh[o + c] = __float2bfloat16_rn(silu_mul(gate_keep[c], v[c]));
            }
        }
    } else if (out_kind == kStoreBF16 && j0 + 16 <= N && (N % 8) == 0) {
        uint32_t w[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * c], v[2 * c + 1]);
            w[c] = *reinterpret_cast<uint32_t*>(&h2);
        }
        const int row0 = i - lane;
        warp_rows_out_bf16(epilogue_stage, w, outh + (size_t)row0 * N + j0, (size_t)N, M - row0, lane, out_policy);
    } else if (out_kind != kStoreBF16 && j0 + 16 <= N && (N % 4) == 0) {
        const int row0 = i - lane;
        warp_rows_out_f32(epilogue_stage, v, outf + (size_t)row0 * N + j0, (size_t)N, M - row0, lane, out_kind == kAddF32, out_policy);
    } else if (i < M && j0 < N) {
        const size_t o = (size_t)i * N + j0;
        const bool full = j0 + 16 <= N;
        if (out_kind == kStoreBF16) {
            if (full && (N % 8) == 0) {
                uint32_t w[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * c], v[2 * c + 1]);
                    w[c] = *reinterpret_cast<uint32_t*>(&h2);
                }
                uint4* dst = reinterpret_cast<uint4*>(outh + o);
                dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
#pragma unroll
                for (int c = 0; c < 16; ++c)
                    if (j0 + c < N) outh[o + c] = __float2bfloat16_rn(v[c]);
            }
        } else if (full && (N % 4) == 0) {
            float4* dst = reinterpret_cast<float4*>(outf + o);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float4 t = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                if (out_kind == kAddF32) {
                    const float4 old = dst[c];
                    t.x += old.x; t.y += old.y; t.z += old.z; t.w += old.w;
                }
                dst[c] = t;
            }
        } else {
#pragma unroll
            for (int c = 0; c < 16; ++c)
                if (j0 + c < N) {
                    if (out_kind == kAddF32) outf[o + c] += v[c]; else outf[o + c] = v[c];
                }
        }
    }
}

}  // namespace tc
}  // namespace citlali
