// Host side of the TMA-fed kernels: tensor maps for row-major bfloat16 matrices.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace citlali {
namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's entry-point query (the library does not link libcuda); nullptr
// if the driver does not provide it.
inline EncodeTiledFn encode_tiled_fn() {
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

// A [rows, row_elems] bfloat16 matrix with a row pitch of `pitch_elems` elements as tiles of [box_rows, 64] with
// 128-byte swizzle; outside the matrix a tile reads zeros.  `who` names the caller in the error text.
//
// A tensor map holds an address and a geometry, no data: the map made for a matrix stays right for as long as a
// matrix of that shape lies at that address.  Encoding one costs the host two to three microseconds, and a step of
// a model makes two for each of its few hundred products, mostly for the same weights and the same recycled
// activation buffers: the maps are kept in a small table by (address, geometry) and found again.
struct MapKey {
    const void* base;
    uint64_t rows, row_elems, pitch_elems;
    int box_rows;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && row_elems == o.row_elems && pitch_elems == o.pitch_elems && box_rows == o.box_rows;
    }
};

inline int make_bf16_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_elems, uint64_t pitch_elems,
                         int box_rows, const char* who) {
    constexpr int kSlots = 2048;                       // direct-mapped; a collision just encodes again
    struct Slot { MapKey key; CUtensorMap map; bool used; };
    static Slot* table = new Slot[kSlots]();
    static std::mutex lock;
    const MapKey key{base, rows, row_elems, pitch_elems, box_rows};
    uint64_t h = (uint64_t)(uintptr_t)base * 0x9E3779B97F4A7C15ull ^ (rows * 0xC2B2AE3D27D4EB4Full) ^ (row_elems << 20) ^
                 (pitch_elems << 7) ^ (uint64_t)box_rows;
    Slot& slot = table[(h >> 17) % kSlots];
    {
        std::lock_guard<std::mutex> guard(lock);
        if (slot.used && slot.key == key) {
            std::memcpy(map, &slot.map, sizeof(CUtensorMap));
            return 0;
        }
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        set_last_error("%s: the driver does not provide cuTensorMapEncodeTiled", who);
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
        set_last_error("%s: cuTensorMapEncodeTiled failed with %d for a [%llu, %llu] matrix at %p", who, (int)r,
                       (unsigned long long)rows, (unsigned long long)row_elems, base);
        return kBadShape;
    }
    {
        std::lock_guard<std::mutex> guard(lock);
        slot.key = key;
        std::memcpy(&slot.map, map, sizeof(CUtensorMap));
        slot.used = true;
    }
    return 0;
}

}  // namespace tc
}  // namespace citlali
