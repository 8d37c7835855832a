#include "tmap.h"

#include <cuda_runtime.h>

#include <mutex>
#include <unordered_map>

namespace s1 {
namespace {

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

struct Key {
    const void* ptr;
    uint64_t rows, cols, stride;
    uint32_t box_rows, box_cols;  // box_cols 0: 64 columns with the 128-byte swizzle
    bool operator==(const Key& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && stride == o.stride && box_rows == o.box_rows &&
               box_cols == o.box_cols;
    }
};
struct Hash {
    size_t operator()(const Key& k) const {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.stride;
        h = h * 1000003u ^ (size_t)k.box_rows;
        h = h * 1000003u ^ (size_t)k.box_cols;
        return h;
    }
};

bool encode(const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride, uint32_t box_rows, uint32_t box_cols,
            CUtensorMap* out) {
    static std::mutex lock;
    static std::unordered_map<Key, CUtensorMap, Hash> cache;
    const Key key{ptr, rows, cols, row_stride, box_rows, box_cols};
    std::lock_guard<std::mutex> hold(lock);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiled fn = encode_fn();
    if (!fn || rows == 0 || cols == 0) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
    const cuuint32_t box[2] = {box_cols ? box_cols : 64u, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap map;
    const CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          box_cols ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return true;
}

}  // namespace

bool tensor_map_2d(const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride, uint32_t box_rows,
                   CUtensorMap* out) {
    return encode(ptr, rows, cols, row_stride, box_rows, 0, out);
}

bool tensor_map_2d_plain(const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride, uint32_t box_rows,
                         uint32_t box_cols, CUtensorMap* out) {
    return encode(ptr, rows, cols, row_stride, box_rows, box_cols, out);
}

}  // namespace s1
