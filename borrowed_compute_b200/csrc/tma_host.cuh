// Host side of TMA: the driver's encoder of tensor maps (asked for once, through the runtime,
// so the library links against no driver stub), and the map of a paged cache.
#pragma once

#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

typedef CUresult (*BcEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

static inline BcEncodeTiledFn bc_encode_tiled_fn() {
    static BcEncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (BcEncodeTiledFn)p;
    });
    return fn;
}

// One plane of a paged cache, [pages][kv heads][64 positions][D] bf16, as a matrix
// [pages * kv heads * 64, D] cut into boxes of 64 positions x 64 elements, 128-byte swizzle:
// the page of (page, kv head) starts at row (page * kv_heads + kv_head) * 64.
static inline int bc_cache_map(CUtensorMap* map, const void* base, long long rows, int D, const char* who) {
    BcEncodeTiledFn enc = bc_encode_tiled_fn();
    if (!enc) {
        bc_set_error("%s: the driver gives no cuTensorMapEncodeTiled", who);
        return BC_ERR_DRIVER;
    }
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, BC_PAGE};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        bc_set_error("%s: cuTensorMapEncodeTiled failed (%d) for a cache of %lld rows of %d", who, (int)r, rows, D);
        return BC_ERR_DRIVER;
    }
    return BC_OK;
}

// Cache maps are made once per (pointer, shape) and kept: the cache's storage does not move.
struct BcCacheKey {
    const void* p;
    long long rows;
    int D;
    bool operator==(const BcCacheKey& o) const { return p == o.p && rows == o.rows && D == o.D; }
};
struct BcCacheKeyHash {
    size_t operator()(const BcCacheKey& k) const { return std::hash<const void*>()(k.p) ^ ((size_t)k.rows * 1000003u) ^ (size_t)k.D; }
};

static inline int bc_cached_cache_map(CUtensorMap* out, const void* base, long long rows, int D, const char* who) {
    static std::unordered_map<BcCacheKey, CUtensorMap, BcCacheKeyHash> maps;   // one a translation unit
    static std::mutex mutex;
    std::lock_guard<std::mutex> lock(mutex);
    BcCacheKey key{base, rows, D};
    auto it = maps.find(key);
    if (it == maps.end()) {
        CUtensorMap m;
        int st = bc_cache_map(&m, base, rows, D, who);
        if (st != BC_OK) return st;
        if (maps.size() > 4096) maps.clear();
        it = maps.emplace(key, m).first;
    }
    *out = it->second;
    return BC_OK;
}
