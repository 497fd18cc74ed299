// Host side of the tensor-map helpers (see tma.cuh).
#include "tma.cuh"
#include "common.cuh"
#include <mutex>
#include <unordered_map>

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool looked = false;
    if (!looked) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        looked = true;
    }
    return fn;
}

int dl_tmap_encode_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                           uint32_t box_rows, uint32_t box_cols, int swizzle) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        dl_fail(DL_ERR_LAUNCH, "tensor map: the driver offers no cuTensorMapEncodeTiled");
        return -1;
    }
    if (((uintptr_t)base % 16) || (pitch_bytes % 16) || ((box_cols * 2) % 16) || box_rows > 256 || box_cols > 256 ||
        (swizzle == DL_TMAP_SWIZZLE_128B && box_cols * 2 != 128)) {
        dl_fail(DL_ERR_ARGUMENT, "tensor map: base %p pitch %llu box %ux%u swizzle %d break the alignment rules", base,
                (unsigned long long)pitch_bytes, box_rows, box_cols, swizzle);
        return -2;
    }
    const cuuint64_t dims[2] = {cols, rows};                  // innermost first
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle == DL_TMAP_SWIZZLE_128B ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        dl_fail(DL_ERR_LAUNCH, "tensor map: cuTensorMapEncodeTiled returned %d (rows %llu cols %llu pitch %llu box %ux%u)",
                (int)r, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)pitch_bytes, box_rows, box_cols);
        return -2;
    }
    return 0;
}

namespace {
struct MapKey {
    const void* base;
    unsigned long long rows, cols, pitch;
    uint32_t box_rows, box_cols;
    int swizzle;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows &&
               box_cols == o.box_cols && swizzle == o.swizzle;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.base);
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.pitch;
        h = h * 1000003u ^ ((size_t)k.box_rows << 20 | (size_t)k.box_cols << 4 | (size_t)k.swizzle);
        return h;
    }
};
}  // namespace

int dl_tmap_cached_2d_bf16(CUtensorMap* out, const void* base, unsigned long long rows, unsigned long long cols,
                           unsigned long long pitch_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
    static std::mutex maps_mutex;
    std::lock_guard<std::mutex> lock(maps_mutex);
    const MapKey key{base, rows, cols, pitch_bytes, box_rows, box_cols, swizzle};
    auto it = maps.find(key);
    if (it == maps.end()) {
        CUtensorMap fresh;
        const int rc = dl_tmap_encode_2d_bf16(&fresh, base, rows, cols, pitch_bytes, box_rows, box_cols, swizzle);
        if (rc != 0) return rc;
        if (maps.size() > 8192) maps.clear();
        it = maps.emplace(key, fresh).first;
    }
    *out = it->second;
    return 0;
}
