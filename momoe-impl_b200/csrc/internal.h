// Internal declarations shared by the translation units of libmomoe_b200.so.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace momoe {

constexpr int TILE_M = 128;  // rows of one expert-major tile; every expert segment is padded to a multiple
constexpr int TILE_K = 64;   // bf16 elements per 128-byte swizzle row
constexpr int UMMA_K = 16;

// Status codes returned by the C entry points (negative: rejected on the host).
enum : int {
    MOMOE_OK = 0,
    MOMOE_ERR_ARG = -1,        // bad pointer / size / alignment
    MOMOE_ERR_UNSUPPORTED = -2,  // shape outside what the kernels handle
    MOMOE_ERR_CUDA = -3,       // a CUDA runtime / driver call failed
    MOMOE_ERR_TOO_LARGE = -4,  // exceeds a fixed capacity
};
// Codes written by kernels into the caller's device status word.
enum : int {
    DEV_TIMEOUT_PRODUCER = 101,
    DEV_TIMEOUT_MMA = 102,
    DEV_TIMEOUT_EPILOGUE = 103,
    DEV_BAD_TOPK_COUNT = 201,   // a token does not have exactly K experts in mask_NM
    DEV_BAD_EXPERT_ID = 202,
    DEV_TIMEOUT_PEER = 301,     // a peer rank did not reach the hand-shake in time
    DEV_EP_OVERFLOW = 302,      // a rank would receive more rows than its buffers hold
};

// sched[] layout (device int32[8]) written by the permutation builder and read by every later kernel.
enum : int { SCHED_N_TILES = 0, SCHED_N_SAVED_TILES = 1, SCHED_PAD_ROWS = 2, SCHED_N_PAIRS = 3, SCHED_WORDS = 8 };

int sm_count();

// Kernels that may run beside a grouped GEMM ask for the same shared-memory / L1 split as the GEMM (everything
// shared): an SM only changes its split while it is idle, so a resident block with another preference keeps the
// GEMM's thread blocks off its SM until it has finished, and the two launches run one after the other.
template <auto Kernel>
static inline void share_sm_with_gemm() {
    static bool done[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return;
    if (!done[dev]) {
        if (cudaFuncSetAttribute(Kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared) != cudaSuccess)
            (void)cudaGetLastError();
        done[dev] = true;
    }
}
// Shared-memory swizzle of a tensor map: the byte span inside which TMA permutes 16-byte chunks.
enum TmapSwizzle : int { TMAP_SWIZZLE_128B = 0, TMAP_SWIZZLE_64B = 1, TMAP_SWIZZLE_32B = 2 };
int encode_tmap_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                   uint32_t box_cols, int swizzle = TMAP_SWIZZLE_128B);
int encode_tmap_3d(CUtensorMap* m, const void* base, uint64_t d2, uint64_t rows, uint64_t cols, uint32_t box_rows,
                   uint32_t box_cols, int swizzle = TMAP_SWIZZLE_128B);
// General form: dims / box innermost first, strides (bytes) of dimensions 1..rank-1.
int encode_tmap(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                const uint32_t* box, int swizzle);

}  // namespace momoe
