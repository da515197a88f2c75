// Host side of the TMA copies: tensor maps over row-major bfloat16 matrices, encoded through the
// driver entry point (no link against libcuda) and kept in a small cache, since the same weight
// and activation buffers come back every step.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

namespace llb_tma {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

struct MapKey {
    const void* ptr; long long rows; int cols, ld, box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        for (long long v : {k.rows, (long long)k.cols, (long long)k.ld, (long long)k.box_rows}) h = h * 1000003u ^ (size_t)v;
        return h;
    }
};

// A 2-D map over a row-major bf16 matrix [rows, cols] with row stride ld (elements): boxes of
// {64 columns, box_rows rows}, 128-byte swizzle, zero fill outside.  The base must be 16-byte
// aligned and ld a multiple of 8.  Returns 0, cudaErrorNotSupported, or -(1000 + CUresult) when
// the encoding is refused.  Encodes into the caller's storage: no cache, no heap.
static inline int encode_bf16_map_64(const void* ptr, long long rows, int cols, int ld, int box_rows, CUtensorMap* out) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -1000 - (int)r;
}

// The same through a cache keyed by pointer and shape.
static inline int bf16_map_64(const void* ptr, long long rows, int cols, int ld, int box_rows, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    MapKey key{ptr, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    int rc = encode_bf16_map_64(ptr, rows, cols, ld, box_rows, out);
    if (rc) return rc;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

// A 2-D map over a row-major float32 matrix [rows, cols] with row stride ld (elements): boxes of {box_cols columns,
// box_rows rows}, no swizzle (a box lies in shared memory as [box_rows][box_cols]); for stores and reductions, which
// clip what lies outside the matrix.  The base must be 16-byte aligned and ld a multiple of 4.  Cached like the others.
static inline int f32_map_plain(const void* ptr, long long rows, int cols, int ld, int box_cols, int box_rows, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    MapKey key{ptr, rows, cols, ld, box_rows * 65536 + box_cols};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -1000 - (int)r;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

}  // namespace llb_tma
