// Host helpers: device properties and TMA tensor-map encoding.
// cuTensorMapEncodeTiled is resolved through the runtime, so the library has no link-time dependency on
// libcuda and loads (for symbol checks) on machines without a driver.
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

// Row-major bf16 matrix [rows, cols]; box = [box_rows, box_cols]; 128-byte swizzle, zero fill outside.
int encode_tmap_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                   uint32_t box_cols) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return MOMOE_ERR_CUDA;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (cols * 2) % 16 != 0) return MOMOE_ERR_ARG;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MOMOE_OK : MOMOE_ERR_CUDA;
}

// Row-major bf16 tensor [d2, rows, cols]; box = [1, box_rows, box_cols].
int encode_tmap_3d(CUtensorMap* m, const void* base, uint64_t d2, uint64_t rows, uint64_t cols, uint32_t box_rows,
                   uint32_t box_cols) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return MOMOE_ERR_CUDA;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (cols * 2) % 16 != 0) return MOMOE_ERR_ARG;
    cuuint64_t dims[3] = {cols, rows, d2};
    cuuint64_t strides[2] = {cols * 2, rows * cols * 2};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MOMOE_OK : MOMOE_ERR_CUDA;
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
