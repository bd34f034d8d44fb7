// Host helpers: device properties and TMA tensor-map encoding.
// cuTensorMapEncodeTiled is resolved through the runtime, so the library has no link-time dependency on
// libcuda and loads (for symbol checks) on machines without a driver.
#include <cstring>
#include <mutex>

#include "internal.h"
#include "../../include/momoe_b200.h"

namespace momoe {

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Tensor maps are cached: encoding one costs about a microsecond of host time, and a layer re-creates the same few
// maps (same buffers from the caching allocator, same shapes) every step.  Direct-mapped table keyed by every input of
// the encoding, guarded by a mutex; an entry is immutable once written.
struct TmapKey {
    const void* base;
    int rank, swizzle;
    uint64_t dims[3];
    uint64_t strides[2];
    uint32_t box[3];
    bool operator==(const TmapKey& o) const {
        return base == o.base && rank == o.rank && swizzle == o.swizzle && memcmp(dims, o.dims, sizeof(dims)) == 0 &&
               memcmp(strides, o.strides, sizeof(strides)) == 0 && memcmp(box, o.box, sizeof(box)) == 0;
    }
};
struct TmapSlot {
    bool used;
    TmapKey key;
    CUtensorMap map;
};
constexpr int TMAP_CACHE_SLOTS = 256;
static TmapSlot g_tmap_cache[TMAP_CACHE_SLOTS];
static std::mutex g_tmap_mu;

static size_t tmap_hash(const TmapKey& k) {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= (k.dims[0] * 31 + k.dims[1]) * 0xC2B2AE3D27D4EB4Full + k.dims[2] * 0x165667B19E3779F9ull;
    h ^= (static_cast<uint64_t>(k.box[0]) << 40) ^ (static_cast<uint64_t>(k.box[1]) << 20) ^ k.box[2] ^
         (static_cast<uint64_t>(k.swizzle) << 60) ^ (static_cast<uint64_t>(k.rank) << 56);
    h ^= h >> 29;
    return static_cast<size_t>(h % TMAP_CACHE_SLOTS);
}

int encode_tmap(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                const uint32_t* box, int swizzle) {
    if (rank < 2 || rank > 3) return MOMOE_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return MOMOE_ERR_ARG;
    TmapKey key;
    memset(&key, 0, sizeof(key));
    key.base = base;
    key.rank = rank;
    key.swizzle = swizzle;
    for (int i = 0; i < rank; ++i) {
        key.dims[i] = dims[i];
        key.box[i] = box[i];
        if (i > 0) {
            if (strides_bytes[i - 1] % 16 != 0) return MOMOE_ERR_ARG;
            key.strides[i - 1] = strides_bytes[i - 1];
        }
    }
    const size_t slot = tmap_hash(key);
    {
        std::lock_guard<std::mutex> lock(g_tmap_mu);
        if (g_tmap_cache[slot].used && g_tmap_cache[slot].key == key) {
            *m = g_tmap_cache[slot].map;
            return MOMOE_OK;
        }
    }
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return MOMOE_ERR_CUDA;
    cuuint64_t d[3], st[2];
    cuuint32_t b[3], estr[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        if (i > 0) st[i - 1] = strides_bytes[i - 1];
    }
    const CUtensorMapSwizzle sw = swizzle == TMAP_SWIZZLE_64B ? CU_TENSOR_MAP_SWIZZLE_64B
                                  : swizzle == TMAP_SWIZZLE_32B ? CU_TENSOR_MAP_SWIZZLE_32B
                                                                : CU_TENSOR_MAP_SWIZZLE_128B;
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, st,
                    b, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return MOMOE_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_tmap_mu);
    g_tmap_cache[slot].used = true;
    g_tmap_cache[slot].key = key;
    g_tmap_cache[slot].map = *m;
    return MOMOE_OK;
}

// Row-major bf16 matrix [rows, cols]; box = [box_rows, box_cols]; zero fill outside.
int encode_tmap_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                   uint32_t box_cols, int swizzle) {
    const uint64_t dims[2] = {cols, rows};
    const uint64_t strides[1] = {cols * 2};
    const uint32_t box[2] = {box_cols, box_rows};
    return encode_tmap(m, base, 2, dims, strides, box, swizzle);
}

// Row-major bf16 tensor [d2, rows, cols]; box = [1, box_rows, box_cols].
int encode_tmap_3d(CUtensorMap* m, const void* base, uint64_t d2, uint64_t rows, uint64_t cols, uint32_t box_rows,
                   uint32_t box_cols, int swizzle) {
    const uint64_t dims[3] = {cols, rows, d2};
    const uint64_t strides[2] = {cols * 2, rows * cols * 2};
    const uint32_t box[3] = {box_cols, box_rows, 1};
    return encode_tmap(m, base, 3, dims, strides, box, swizzle);
}

}  // namespace momoe

extern "C" __attribute__((visibility("default"))) int momoe_version(void) { return 100; }

extern "C" __attribute__((visibility("default"))) int64_t momoe_tile_capacity(int32_t M, int32_t K, int32_t N) {
    // every expert adds at most one partially filled tile
    const int64_t msum = static_cast<int64_t>(M) * K;
    return (msum + momoe::TILE_M - 1) / momoe::TILE_M + N;
}

extern "C" __attribute__((visibility("default"))) int64_t momoe_sorted_rows_capacity(int32_t M, int32_t K, int32_t N) {
    return momoe_tile_capacity(M, K, N) * momoe::TILE_M;
}
