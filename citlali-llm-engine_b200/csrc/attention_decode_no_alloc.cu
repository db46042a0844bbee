// The allocation-free variant of split-context decode attention: see no_alloc.h for who needs
// it, its limit and its rules.  The scratch array, the lookup of its device address and the
// entry point are all in this file, because the array's name means two different things: in
// device code it is the array; in host code it is only a handle that cudaGetSymbolAddress
// turns into the device address.  Passing the bare name to a kernel from host code would hand
// the kernel a host-side address.
#include "no_alloc.h"

#include "api.h"
#include "common.cuh"

#include <atomic>

namespace citlali {

static __device__ __align__(256) float g_no_alloc_scratch[CITLALI_NO_ALLOC_SCRATCH_FLOATS];
// Counters of the kernel that deals long rows out by length: zero when the library is loaded, and every call
// leaves them zero.
static __device__ __align__(256) int g_no_alloc_counters[CITLALI_NO_ALLOC_COUNTER_INTS];

// Device code may name the array directly.  This kernel is never launched; it keeps the array
// in the device image even though no other device code in this file refers to it.
__global__ void no_alloc_scratch_anchor(float* out) {
    if (out != nullptr) out[0] = g_no_alloc_scratch[0] + (float)g_no_alloc_counters[0];
}

constexpr int kMaxDevices = 64;
// One address per device.  Two host threads that make their first call on a device at the same time
// both look the address up and both store the same value: harmless, and the slot is atomic so that
// neither reads a torn pointer.
static std::atomic<float*> g_scratch_address[kMaxDevices];
static std::atomic<int*> g_counters_address[kMaxDevices];

// The device address of the array on the current device; looked up on the first call per device.
static int scratch_for_current_device(float** ptr, int** counters) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= kMaxDevices) {
        set_last_error("attention_decode_no_alloc: device index %d is outside 0..%d", device, kMaxDevices - 1);
        return kBadShape;
    }
    float* known = g_scratch_address[device].load(std::memory_order_acquire);
    if (known == nullptr) {
        float* address = nullptr;
        e = cudaGetSymbolAddress((void**)&address, g_no_alloc_scratch);
        if (e != cudaSuccess) {
            set_last_error("attention_decode_no_alloc: cudaGetSymbolAddress failed on device %d: %s", device,
                           cudaGetErrorString(e));
            return (int)e;
        }
        g_scratch_address[device].store(address, std::memory_order_release);
        known = address;
    }
    int* known_counters = g_counters_address[device].load(std::memory_order_acquire);
    if (known_counters == nullptr) {
        int* address = nullptr;
        e = cudaGetSymbolAddress((void**)&address, g_no_alloc_counters);
        if (e != cudaSuccess) {
            set_last_error("attention_decode_no_alloc: cudaGetSymbolAddress (counters) failed on device %d: %s", device,
                           cudaGetErrorString(e));
            return (int)e;
        }
        g_counters_address[device].store(address, std::memory_order_release);
        known_counters = address;
    }
    *ptr = known;
    *counters = known_counters;
    return 0;
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_attention_decode_no_alloc(const void* q, int q_stride, const void* k_pool, const void* v_pool,
                                                 const int32_t* page_table, int page_table_stride,
                                                 const int32_t* row_slot, const int32_t* row_pos,
                                                 void* out, int out_stride,
                                                 int rows, int nq, int nkv, int head_dim, int page_size, int window,
                                                 int max_positions, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (nq <= 0 || head_dim <= 0 || page_size <= 0 || max_positions <= 0) {
        set_last_error("attention_decode_no_alloc: sizes must be positive (heads %d, head size %d, page %d, positions %d)",
                       nq, head_dim, page_size, max_positions);
        return kBadShape;
    }
    const size_t need = citlali_attention_decode_scratch_floats(rows, nq, head_dim, page_size, max_positions);
    if (need > (size_t)CITLALI_NO_ALLOC_SCRATCH_FLOATS) {
        set_last_error("attention_decode_no_alloc: %d rows x %d heads x head size %d over %d positions need %zu floats of "
                       "scratch; the built-in array holds %u (use citlali_attention_decode with your own scratch)",
                       rows, nq, head_dim, max_positions, need, (unsigned)CITLALI_NO_ALLOC_SCRATCH_FLOATS);
        return kTooLarge;
    }
    // one counter per row and group of 16 query heads of a key/value head: never more than rows * nq
    if ((size_t)rows * (size_t)nq > (size_t)CITLALI_NO_ALLOC_COUNTER_INTS) {
        set_last_error("attention_decode_no_alloc: %d rows x %d heads exceed the %u built-in counters", rows, nq,
                       (unsigned)CITLALI_NO_ALLOC_COUNTER_INTS);
        return kTooLarge;
    }
    float* scratch = nullptr;
    int* counters = nullptr;
    const int rc = scratch_for_current_device(&scratch, &counters);
    if (rc) return rc;
    return citlali_attention_decode(q, q_stride, k_pool, v_pool, page_table, page_table_stride, row_slot, row_pos, out,
                                    out_stride, scratch, (size_t)CITLALI_NO_ALLOC_SCRATCH_FLOATS, counters,
                                    (size_t)CITLALI_NO_ALLOC_COUNTER_INTS, rows, nq, nkv, head_dim,
                                    page_size, window, max_positions, scale, stream);
}
