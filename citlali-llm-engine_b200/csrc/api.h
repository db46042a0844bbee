// The C interface of the kernel library.  Every function launches on the given stream and
// returns 0, a cudaError_t (> 0), or a refusal (< 0) whose text citlali_last_error() gives.
// dtype codes: 0 = float32, 1 = bfloat16.  All sizes are in elements unless named bytes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* citlali_last_error(void);

// 1 (default): kernels are launched so that they may start before the kernel before them has
// finished, and wait for it on the device; 0: plain stream order.
void citlali_set_dependent_launch(int enabled);

// out[m, :] = table[tokens[m], :] widened to float32 and multiplied by `scale` (1: a plain row copy).
int citlali_embed_rows(const void* table, int table_dtype, const int32_t* tokens, float* out,
                       int rows, int hidden, int vocab, float scale, int32_t* error_flag, cudaStream_t stream);

// rows_out = bfloat16(x) [rows, hidden] and sumsq[r, g] = sum of x[r, 32 g .. 32 g + 31]^2 (hidden a multiple of 32):
// what citlali_gemm_tc_normed's `scale_sumsq` reads, for rows that did not come out of an emitting product.
int citlali_norm_inputs(const float* x, void* rows_out, float* sumsq, int rows, int hidden, cudaStream_t stream);

// x[0..n) *= scale.
int citlali_scale(float* x, size_t n, float scale, cudaStream_t stream);

// out[r, :] = x[idx[r], :] * rsqrt(mean(x^2) + eps) * gain   (idx may be null: identity).
int citlali_rms_norm(const float* x, const void* gain, int gain_dtype, const int32_t* row_index,
                     void* out, int out_dtype, int rows, int hidden, float eps, cudaStream_t stream);

// act[m, i] = silu(gate) * up, gate/up taken from one [rows, 2*inter] matrix whose columns
// alternate in runs of `run`: gate run, up run, gate run, ...
int citlali_swiglu(const void* gate_up, void* act, int dtype, int rows, int inter, int run,
                   cudaStream_t stream);

// y[M, N] = x[M, K] . w[N, K]^T on CUDA cores with float accumulation, k ascending.
// accumulate != 0: y (float32) += product.
int citlali_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype,
                      int M, int N, int K, int accumulate, cudaStream_t stream);

// In place on a [rows, (nq + 2 nkv) d] projection: per-head RMSNorm of q and k, half-split
// rotation by the row's position, then k and v written to the paged cache of the row's slot.
// The first `rotary_dim` elements of a head are rotated in pairs (i, i + rotary_dim/2), the rest pass through.
// write_cache: 0 leaves the cache alone (a layer that reads another layer's cache); 1 stores k and v; 2 writes
// the normed, rotated k back into the row instead and leaves v alone (a second call then stores them).
int citlali_qk_norm_rope_cache(void* qkv, int dtype, const void* q_gain, const void* k_gain, int gain_dtype,
                               const float* inv_freq, int rotary_dim,
                               const int32_t* row_slot, const int32_t* row_pos,
                               const int32_t* page_table, int page_table_stride,
                               void* k_pool, void* v_pool, int cache_dtype, int page_size,
                               int rows, int nq, int nkv, int head_dim, float eps, int write_cache,
                               cudaStream_t stream);

// Causal attention of every row over the cache of its slot: keys lo..pos, lo = 0 or
// pos - window + 1.  One order of operations for prompts and for single tokens.
int citlali_attention_rows(const void* q, int q_stride, int dtype,
                           const void* k_pool, const void* v_pool, int cache_dtype,
                           const int32_t* page_table, int page_table_stride,
                           const int32_t* row_slot, const int32_t* row_pos,
                           void* out, int out_stride, int rows, int nq, int nkv, int head_dim,
                           int page_size, int window, int max_keys, float scale,
                           cudaStream_t stream);

// Attention of single new tokens (bfloat16) split over the context; positions are read on the
// device, `max_positions` bounds them and fixes the grid.  `partial` is float scratch of
// citlali_attention_decode_scratch_floats(...) elements.  `counters` (may be nullptr): `counter_ints` 32-bit
// words, at least rows * nkv * ceil((nq / nkv) / 16), zero before the first call; every call leaves them zero.
// With them, a step of many rows deals the pages of its long rows out to several blocks by the rows' lengths.
size_t citlali_attention_decode_scratch_floats(int rows, int nq, int head_dim, int page_size, int max_positions);
int citlali_attention_decode(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                             const int32_t* page_table, int page_table_stride,
                             const int32_t* row_slot, const int32_t* row_pos,
                             void* out, int out_stride, float* partial, size_t partial_floats,
                             int32_t* counters, size_t counter_ints,
                             int rows, int nq, int nkv, int head_dim, int page_size, int window,
                             int max_positions, float scale, cudaStream_t stream);
void citlali_attention_decode_set_split(int split);
void citlali_attention_decode_set_by_length(int on, int run_scale_q8);
void citlali_attention_decode_set_per_warp(int on);

// Causal attention of runs of new tokens (bfloat16, pages of 64) on the tensor cores.  Sequence b
// owns rows seq_start[b] .. seq_start[b+1]-1 at positions seq_past[b] + i of slot seq_slot[b].
int citlali_attention_prefill_supports(int head_dim, int page_size);
int citlali_attention_prefill(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                              const int32_t* page_table, int page_table_stride,
                              const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_past,
                              void* out, int out_stride, int sequences, int max_new,
                              int nq, int nkv, int head_dim, int page_size, int window, float scale,
                              cudaStream_t stream);

// The same on tcgen05 (scores and output in tensor memory), for head size 128 and pages of 64.
// total_rows: rows of q over all sequences; pool_pages: pages of the layer's key and value pools.
int citlali_attention_prefill_tc_supports(int head_dim, int page_size);
int citlali_attention_prefill_tc(const void* q, int q_stride, int total_rows,
                                 const void* k_pool, const void* v_pool, int pool_pages,
                                 const int32_t* page_table, int page_table_stride,
                                 const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_past,
                                 void* out, int out_stride, int sequences, int max_new,
                                 int nq, int nkv, int head_dim, int page_size, int window, float scale,
                                 int32_t* error_flag, cudaStream_t stream);

// tokens[r] = argmax of logits[r, :] over finite values, lowest index on ties.
int citlali_argmax_rows(const float* logits, int32_t* tokens, int rows, int vocab, cudaStream_t stream);
// The same with 64 blocks per row; scratch holds rows * 128 floats.
int citlali_argmax_rows_wide(const float* logits, int32_t* tokens, float* scratch, int rows, int vocab,
                             cudaStream_t stream);

// tokens[r] = first index whose inclusive CDF of softmax(logits[r] / temperature[r]) exceeds
// uniform[r]; temperature[r] <= 0 means argmax.
int citlali_sample_rows(const float* logits, const float* temperature, const float* uniform,
                        int32_t* tokens, int rows, int vocab, cudaStream_t stream);

// The tensor-core product (bfloat16 operands, float accumulation).  citlali_gemm_tc_plan tells
// how a shape runs: whether the weights are the 128-row operand (*swapped), the narrow tile
// (*bn) and the K split (*splits).  force_splits > 0 replaces the plan's split (at most 8).
int citlali_gemm_tc_plan(int M, int N, int K, int sm_count, int force_splits, int* swapped, int* bn, int* splits);
// y = x[M, K] . w[N, K]^T.  mode bits: 1 = y (float32) += product; 2 = SiLU-gate epilogue (w's rows
// alternate in runs of 16 between gate and up; y is bfloat16 [M, N/2]).  K must be a multiple of 8
// and the operands 16-byte aligned.  A shape that splits K runs each tile's splits as a cluster
// that sums its partials through distributed shared memory, in split order; no scratch is needed.
// error_flag[1..2] receive the code and block of a wait that ran out.
int citlali_gemm_tc(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                    int mode, int force_splits, int32_t* error_flag, int sm_count, cudaStream_t stream);
// The same for few rows of x with a layer norm's work in the epilogue (gemm_tcgen05.cu says what each pointer means;
// null pointers: plain citlali_gemm_tc).
int citlali_gemm_tc_normed(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                           int mode, int force_splits, int32_t* error_flag, int sm_count,
                           void* emit_rows, float* emit_sumsq, const float* scale_sumsq, int scale_groups,
                           int scale_dim, float scale_eps, cudaStream_t stream);
// The same product on pairs of SMs (tcgen05.mma with cta_group::2: a [256 x BN] tile per cluster of two
// blocks, each fetching half of both operands).  With equal waves it takes 0.92-0.97 of the one-block
// kernel's time at 512 to 4,096 rows and 0.82 at 8,192, and it loses where its 256-row tiles need a wave
// more.  citlali_gemm_tc uses it from citlali_gemm_tc_set_pair_rows' number of rows on (512 unless set;
// 0: never; the call returns the number that stood before) where the waves of pairs cost less, on devices
// that run such clusters; citlali_gemm_tc_runs_on_pairs says whether a shape goes there, and
// citlali_gemm_tc_pair_plan gives the tile width and the pairs that run at once.
int citlali_gemm_tc_pair(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                         int mode, int32_t* error_flag, cudaStream_t stream);
int citlali_gemm_tc_pair_plan(int M, int N, int K, int* bn, int* pairs);
// Many rows: the row tiles run in bands whose rows of x (this many bytes, default 32 MiB) stay in L2 while all
// weight tiles pass by.  Sets the size and returns the one before (for tuning).
long citlali_gemm_tc_pair_set_band_bytes(long bytes);
int citlali_gemm_tc_set_pair_rows(int rows);
// The kernels' bounded wait on its own: a block waits `limit_ns` (at most one second) on a barrier on which
// nothing arrives, gives up, records code 900 in error_flag[1] and its block in error_flag[2], and leaves
// normally; result[0] = the wait's return value (0), result[1] = the block's abort word (1).
int citlali_wait_selftest(int32_t* error_flag, int* result, long long limit_ns, cudaStream_t stream);
int citlali_gemm_tc_runs_on_pairs(int M, int N, int K, int sm_count, int gate_runs);

#ifdef __cplusplus
}
#endif
