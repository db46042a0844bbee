// citlali_attention_decode_no_alloc: split-context attention of single new tokens for callers
// that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (xissleah/Citlali-LLM-Engine allocates
// every buffer with cudaMalloc at load time and has no split-context attention).  It exists
// for hosts that drive the kernel library from a place where allocation is impossible or
// forbidden: code running inside a CUDA stream capture (cudaMalloc is illegal there), a
// real-time or embedded loop that was handed a fixed memory budget and may not touch the
// allocator, or a foreign runtime (another language's FFI, a plugin sandbox) that can pass
// pointers it already owns but has no way to obtain new device memory for scratch.
//
// It computes exactly what citlali_attention_decode computes, with the same kernels, but the
// float scratch that holds the per-chunk partial results lives in a fixed array inside the
// library instead of being passed in, and so do the counters that a step of many rows uses.
// (For pages of 64 keys, the head sizes of the tensor-core kernel and few rows the blocks
// exchange their partial results through shared memory and the arrays are not touched; the
// limit below is checked all the same.)
//
//   Limit.  The array holds CITLALI_NO_ALLOC_SCRATCH_FLOATS floats (4 MiB).  A call needs
//   rows * nq * ceil(max_positions / (2 * page_size)) * (head_dim + 2) floats; a call that
//   needs more is refused with a negative return code and a message (citlali_last_error),
//   and nothing is launched.  Every GPU that loads the library holds these 4 MiB until the
//   process exits.  Beside it lie CITLALI_NO_ALLOC_COUNTER_INTS 32-bit counters (256 KiB), one
//   per row and group of query heads; a call of more rows x heads than that is refused likewise.
//
//   First call.  The first call on each device looks up the array's device address
//   (cudaGetSymbolAddress) and remembers it.  Make that first call outside any stream
//   capture, with the device that will run the kernels current.  Host threads may make their
//   first calls at the same time: each looks the same address up, and the slot that keeps it is
//   atomic.
//
//   Sharing.  All calls on a device share the one array, and it keeps whatever the last call
//   left in it.  Nothing in it has to start at zero: every partial a call reads was written by
//   that same call first.  The counters are zero when the library is loaded, and every call
//   that finishes leaves them zero.  But two calls whose kernels overlap on the GPU (different
//   streams, or graphs replayed concurrently) race on both; issue them on one stream, or
//   order them.
//
//   It calls no cudaMalloc, cudaFree or any other allocating routine.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define CITLALI_NO_ALLOC_SCRATCH_FLOATS (1u << 20)
#define CITLALI_NO_ALLOC_COUNTER_INTS (1u << 16)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as citlali_attention_decode (api.h), without the scratch and counter pointers and their sizes.
int citlali_attention_decode_no_alloc(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                                      const int32_t* page_table, int page_table_stride,
                                      const int32_t* row_slot, const int32_t* row_pos,
                                      void* out, int out_stride,
                                      int rows, int nq, int nkv, int head_dim, int page_size, int window,
                                      int max_positions, float scale, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
