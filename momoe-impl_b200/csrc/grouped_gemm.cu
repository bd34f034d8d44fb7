// Persistent grouped GEMM for sm_100a: TMA -> shared-memory ring -> tcgen05.mma (accumulators in TMEM) ->
// epilogue warps.  One kernel template serves the five GEMMs of the MoMoE layer; they differ in operand
// majorness, tile width and epilogue.
//
// CTA = 192 threads: warp 0 (one lane) issues TMA loads, warp 1 allocates TMEM and (one lane) issues the MMAs,
// warps 2..5 read accumulators out of TMEM (each warp owns the 32 TMEM lanes of its quarter, warp_id % 4) and
// write the results.  Two accumulator buffers in TMEM let the epilogue of one tile overlap the main loop of
// the next.  Every wait on an mbarrier is bounded (ptx.cuh); a wait that runs out records a code in the
// caller's status word and every role leaves its loop.
//
// Shared-memory operand layouts (all 128-byte swizzled, as written by TMA with SWIZZLE_128B):
//   K-major operand  [R rows x 64 k]: row r at byte r*128; descriptor SBO = 1024 (8-row group pitch);
//                    one MMA (k = 16) advances the start address by 32 bytes.
//   MN-major operand [64 k x 64 mn] boxes of 8 KiB: k-row at byte k*128, boxes along mn 8192 bytes apart;
//                    descriptor LBO = 8192 (mn pitch), SBO = 1024 (8-k group pitch); one MMA advances 2048 bytes.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "internal.h"
#include "ptx.cuh"
#include "../../include/momoe_b200.h"

namespace momoe {

enum GemmMode : int { MODE_UP = 0, MODE_DOWN = 1, MODE_DGRAD2 = 2, MODE_DGRAD1 = 3, MODE_WGRAD = 4 };

struct GemmArgs {
    const int* sched;
    const int* tile_expert;
    const int* pad_off;
    int* status;
    int n_experts;
    int n_nblk;      // column blocks per row tile (row-tile modes) or per output row block (wgrad)
    int n_mblk;      // wgrad: row blocks of one expert's output matrix
    int nkb;         // row-tile modes: k-blocks of 64
    int out_cols;    // valid output columns: H (up, dgrad2), D (down, dgrad1), Y (wgrad)
    int out_rows;    // wgrad: X
    int half;        // up: H, the column where the gate half of W1 starts
    int ab_mode;     // up: 0 none, 1 save tiles < n_saved, 2 recompute tiles >= n_saved
    __nv_bfloat16* out0;
    __nv_bfloat16* out1;
    __nv_bfloat16* out2;
    const float* row_weight;
    const __nv_bfloat16* a_saved;
    const __nv_bfloat16* b_saved;
    const __nv_bfloat16* a_recomp;
    const __nv_bfloat16* b_recomp;
    float* gs_part;
    uint32_t mn_lbo, mn_sbo;  // MN-major descriptor byte offsets
};

template <int MODE>
struct Cfg {
    static constexpr bool A_MN = (MODE == MODE_WGRAD);
    static constexpr bool B_MN = (MODE == MODE_UP || MODE == MODE_DOWN || MODE == MODE_WGRAD);
    static constexpr int BN = (MODE == MODE_DGRAD2) ? 128 : 256;
    static constexpr int A_BYTES = TILE_M * TILE_K * 2;   // 16 KiB
    static constexpr int B_BYTES = BN * TILE_K * 2;       // 16 or 32 KiB
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN == 256) ? 4 : 6;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;  // + slack for 1024-byte alignment
    static constexpr int ACC_BUFS = 2;
    static constexpr int TMEM_COLS = 512;
};

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ void unpack_bf16(uint32_t v, float& lo, float& hi) {
    lo = __uint_as_float(v << 16);
    hi = __uint_as_float(v & 0xFFFF0000u);
}
__device__ __forceinline__ float sigmoidf_fast(float x) { return __frcp_rn(1.0f + __expf(-x)); }

// Store 32 consecutive fp32 values as bf16 to dst (16-byte aligned), keeping only columns < ncols_left.
// ncols_left is a multiple of 8 by contract (all matrix widths are).
__device__ __forceinline__ void store_row32(__nv_bfloat16* dst, const float (&v)[32], int ncols_left) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        if (g * 8 < ncols_left) {
            uint4 q;
            q.x = pack_bf16(v[g * 8 + 0], v[g * 8 + 1]);
            q.y = pack_bf16(v[g * 8 + 2], v[g * 8 + 3]);
            q.z = pack_bf16(v[g * 8 + 4], v[g * 8 + 5]);
            q.w = pack_bf16(v[g * 8 + 6], v[g * 8 + 7]);
            *reinterpret_cast<uint4*>(dst + g * 8) = q;
        }
    }
}
// Load 32 consecutive bf16 values (16-byte aligned) as fp32; columns >= ncols_left read as zero.
__device__ __forceinline__ void load_row32(const __nv_bfloat16* src, float (&v)[32], int ncols_left) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 q = make_uint4(0, 0, 0, 0);
        if (g * 8 < ncols_left) q = __ldg(reinterpret_cast<const uint4*>(src + g * 8));
        unpack_bf16(q.x, v[g * 8 + 0], v[g * 8 + 1]);
        unpack_bf16(q.y, v[g * 8 + 2], v[g * 8 + 3]);
        unpack_bf16(q.z, v[g * 8 + 4], v[g * 8 + 5]);
        unpack_bf16(q.w, v[g * 8 + 6], v[g * 8 + 7]);
    }
}

// Work item -> coordinates.  Row-tile modes: item = tile * n_nblk + nb.  Wgrad: item = (e * n_mblk + mb) * n_nblk + nb.
struct Work {
    int tile;   // row tile (row-tile modes)
    int e;      // expert
    int mb;     // wgrad: output row block
    int nb;     // column block
    int nkb;    // k-blocks
    int row0;   // wgrad: first padded row of the expert
};

template <int MODE>
__device__ __forceinline__ Work decode_work(const GemmArgs& g, int item, int first_tile) {
    Work w;
    if constexpr (MODE == MODE_WGRAD) {
        w.nb = item % g.n_nblk;
        const int t = item / g.n_nblk;
        w.mb = t % g.n_mblk;
        w.e = t / g.n_mblk;
        w.tile = 0;
        w.row0 = __ldg(g.pad_off + w.e);
        w.nkb = (__ldg(g.pad_off + w.e + 1) - w.row0) / TILE_K;
    } else {
        w.nb = item % g.n_nblk;
        w.tile = first_tile + item / g.n_nblk;
        w.e = __ldg(g.tile_expert + w.tile);
        w.mb = 0;
        w.nkb = g.nkb;
        w.row0 = 0;
    }
    return w;
}

template <int MODE>
__global__ void __launch_bounds__(192, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmArgs g) {
    using C = Cfg<MODE>;
    constexpr int BN = C::BN;
    constexpr int STAGES = C::STAGES;

    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[STAGES];
    __shared__ uint64_t bar_empty[STAGES];
    __shared__ uint64_t bar_acc_full[C::ACC_BUFS];
    __shared__ uint64_t bar_acc_empty[C::ACC_BUFS];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t stage_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

    // ---- work range (device-resident schedule; nothing is read back by the host)
    int first_tile = 0;
    int total_items;
    if constexpr (MODE == MODE_WGRAD) {
        total_items = g.n_experts * g.n_mblk * g.n_nblk;
    } else {
        const int n_tiles = __ldg(g.sched + SCHED_N_TILES);
        if (MODE == MODE_UP && g.ab_mode == 2) first_tile = __ldg(g.sched + SCHED_N_SAVED_TILES);
        total_items = (n_tiles - first_tile) * g.n_nblk;
    }
    if (total_items <= 0 || static_cast<int>(blockIdx.x) >= total_items) return;  // whole CTA leaves together

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int b = 0; b < C::ACC_BUFS; ++b) {
            mbar_init(smem_u32(&bar_acc_full[b]), 1);
            mbar_init(smem_u32(&bar_acc_empty[b]), 4);  // one arrival per epilogue warp
        }
        fence_mbar_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
    volatile int* abortp = &abort_flag;

    if (warp == 0) {
        // ================================================================ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
                const Work w = decode_work<MODE>(g, item, first_tile);
                for (int kb = 0; kb < w.nkb; ++kb) {
                    ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp, g.status, DEV_TIMEOUT_PRODUCER);
                    if (!ok) break;
                    const uint32_t sa = stage_base + stage * C::STAGE_BYTES;
                    const uint32_t sb = sa + C::A_BYTES;
                    const uint32_t full = smem_u32(&bar_full[stage]);
                    mbar_arrive_expect_tx(full, C::STAGE_BYTES);
                    if constexpr (MODE == MODE_WGRAD) {
                        const int r0 = w.row0 + kb * TILE_K;
#pragma unroll
                        for (int i = 0; i < TILE_M / 64; ++i)
                            tma_load_2d(sa + i * 8192, &tmA, full, w.mb * TILE_M + i * 64, r0);
#pragma unroll
                        for (int i = 0; i < BN / 64; ++i)
                            tma_load_2d(sb + i * 8192, &tmB, full, w.nb * BN + i * 64, r0);
                    } else {
                        tma_load_2d(sa, &tmA, full, kb * TILE_K, w.tile * TILE_M);
                        if constexpr (MODE == MODE_UP) {
                            // 4 boxes of 64 columns: two from the linear half, two from the gate half of W1[e]
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int col = (i < 2 ? 0 : g.half) + w.nb * 128 + (i & 1) * 64;
                                tma_load_3d(sb + i * 8192, &tmB, full, col, kb * TILE_K, w.e);
                            }
                        } else if constexpr (MODE == MODE_DOWN) {
#pragma unroll
                            for (int i = 0; i < BN / 64; ++i)
                                tma_load_3d(sb + i * 8192, &tmB, full, w.nb * BN + i * 64, kb * TILE_K, w.e);
                        } else {
                            // K-major weights: rows = output columns, 64 contiguous k per row
                            tma_load_3d(sb, &tmB, full, kb * TILE_K, w.nb * BN, w.e);
                        }
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, BN, C::A_MN, C::B_MN);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x, ++it) {
                const Work w = decode_work<MODE>(g, item, first_tile);
                const int ab = it & 1;
                const uint32_t aphase = (it >> 1) & 1u;
                ok = mbar_wait(smem_u32(&bar_acc_empty[ab]), aphase ^ 1u, abortp, g.status, DEV_TIMEOUT_MMA);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + ab * BN;
                for (int kb = 0; kb < w.nkb; ++kb) {
                    ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abortp, g.status, DEV_TIMEOUT_MMA);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = stage_base + stage * C::STAGE_BYTES;
                    const uint32_t sb = sa + C::A_BYTES;
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k) {
                        const uint64_t da = C::A_MN ? umma_smem_desc(sa + k * 2048, g.mn_lbo, g.mn_sbo)
                                                    : umma_smem_desc(sa + k * 32, 16, 1024);
                        const uint64_t db = C::B_MN ? umma_smem_desc(sb + k * 2048, g.mn_lbo, g.mn_sbo)
                                                    : umma_smem_desc(sb + k * 32, 16, 1024);
                        umma_bf16(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&bar_empty[stage]));  // frees the stage once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if (w.nkb > 0) umma_commit(smem_u32(&bar_acc_full[ab]));
                else mbar_arrive(smem_u32(&bar_acc_full[ab]));  // nothing to accumulate: epilogue writes zeros
            }
        }
    } else {
        // ================================================================ epilogue (warps 2..5)
        const int q = warp & 3;            // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;     // accumulator row == TMEM lane
        int it = 0;
        bool ok = true;
        for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x, ++it) {
            const Work w = decode_work<MODE>(g, item, first_tile);
            const int ab = it & 1;
            const uint32_t aphase = (it >> 1) & 1u;
            ok = mbar_wait(smem_u32(&bar_acc_full[ab]), aphase, abortp, g.status, DEV_TIMEOUT_EPILOGUE);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * BN;
            uint32_t r[32];
            float v[32];

            if constexpr (MODE == MODE_UP) {
                const size_t grow = static_cast<size_t>(w.tile) * TILE_M + row;
                const int n_saved = __ldg(g.sched + SCHED_N_SAVED_TILES);
                const bool store_ab = (g.ab_mode == 1 && w.tile < n_saved) || g.ab_mode == 2;
                const size_t abrow =
                    (g.ab_mode == 2 ? static_cast<size_t>(w.tile - n_saved) : static_cast<size_t>(w.tile)) * TILE_M + row;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    const int col0 = w.nb * 128 + c * 32;
                    const int left = g.out_cols - col0;
                    if (left <= 0) break;   // uniform across the warp
                    float a[32], b[32];
                    tmem_ld32(taddr + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) a[i] = __uint_as_float(r[i]);
                    tmem_ld32(taddr + 128 + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) b[i] = __uint_as_float(r[i]);
                    if (store_ab) {
                        store_row32(g.out1 + abrow * g.out_cols + col0, a, left);
                        store_row32(g.out2 + abrow * g.out_cols + col0, b, left);
                    }
                    if (g.out0 != nullptr) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = b[i] * sigmoidf_fast(b[i]) * a[i];
                        store_row32(g.out0 + grow * g.out_cols + col0, v, left);
                    }
                }
            } else if constexpr (MODE == MODE_DOWN || MODE == MODE_DGRAD1) {
                const size_t grow = static_cast<size_t>(w.tile) * TILE_M + row;
                float wgt = 1.0f;
                if constexpr (MODE == MODE_DOWN) wgt = __ldg(g.row_weight + grow);
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int col0 = w.nb * BN + c * 32;
                    const int left = g.out_cols - col0;
                    if (left <= 0) break;
                    tmem_ld32(taddr + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * wgt;
                    store_row32(g.out0 + grow * g.out_cols + col0, v, left);
                }
            } else if constexpr (MODE == MODE_DGRAD2) {
                const size_t grow = static_cast<size_t>(w.tile) * TILE_M + row;
                const int n_saved = __ldg(g.sched + SCHED_N_SAVED_TILES);
                const bool saved = w.tile < n_saved;
                const size_t abrow = (saved ? static_cast<size_t>(w.tile) : static_cast<size_t>(w.tile - n_saved)) * TILE_M + row;
                const __nv_bfloat16* ap = (saved ? g.a_saved : g.a_recomp) + abrow * g.out_cols;
                const __nv_bfloat16* bp = (saved ? g.b_saved : g.b_recomp) + abrow * g.out_cols;
                const float wgt = __ldg(g.row_weight + grow);
                const int H = g.out_cols;
                float gs = 0.0f;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int col0 = w.nb * BN + c * 32;
                    const int left = H - col0;
                    if (left <= 0) break;
                    float a[32], b[32];
                    load_row32(ap + col0, a, left);
                    load_row32(bp + col0, b, left);
                    tmem_ld32(taddr + c * 32, r);
                    tmem_ld_wait();
                    float z1[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float gh_raw = __uint_as_float(r[i]);
                        const float sg = sigmoidf_fast(b[i]);
                        const float hh = bf16_round(a[i] * b[i] * sg);
                        gs += gh_raw * hh;
                        const float gh = wgt * gh_raw;
                        z1[i] = gh * b[i] * sg;
                        v[i] = gh * a[i] * sg * (1.0f + b[i] * (1.0f - sg));   // gate-half gradient
                        a[i] = wgt * hh;                                        // reuse a[] for hs
                    }
                    store_row32(g.out0 + grow * (2 * H) + col0, z1, left);
                    store_row32(g.out0 + grow * (2 * H) + H + col0, v, left);
                    store_row32(g.out1 + grow * H + col0, a, left);
                }
                g.gs_part[grow * g.n_nblk + w.nb] = gs;
            } else {  // MODE_WGRAD
                const int orow = w.mb * TILE_M + row;
                __nv_bfloat16* dst = g.out0 + (static_cast<size_t>(w.e) * g.out_rows + orow) * g.out_cols;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int col0 = w.nb * BN + c * 32;
                    const int left = g.out_cols - col0;
                    if (left <= 0) break;
                    if (w.nkb > 0) {
                        tmem_ld32(taddr + c * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0.0f;
                    }
                    if (orow < g.out_rows) store_row32(dst + col0, v, left);
                }
            }
            // hand the accumulator buffer back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[ab]));
        }
    }

    // ---- teardown: everybody meets, then the allocating warp frees TMEM
    tc_fence_before();
    __syncthreads();
    if (*abortp) {
        // a wait was abandoned: give loads still in flight time to land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------- host side
static int check_plan(const momoe_plan_t* p) {
    if (p == nullptr || p->sched == nullptr || p->tile_expert == nullptr || p->pad_off == nullptr ||
        p->row_weight == nullptr || p->status == nullptr)
        return MOMOE_ERR_ARG;
    if (p->M <= 0 || p->N <= 0 || p->K <= 0 || p->D <= 0 || p->H <= 0 || p->rows_capacity <= 0) return MOMOE_ERR_ARG;
    if (p->D % 8 != 0 || p->H % 8 != 0) return MOMOE_ERR_UNSUPPORTED;  // TMA row pitch must be a multiple of 16 bytes
    if (p->rows_capacity % TILE_M != 0) return MOMOE_ERR_ARG;
    return MOMOE_OK;
}

static void base_args(const momoe_plan_t* p, GemmArgs& g) {
    memset(&g, 0, sizeof(g));
    g.sched = p->sched;
    g.tile_expert = p->tile_expert;
    g.pad_off = p->pad_off;
    g.status = p->status;
    g.n_experts = p->N;
    g.row_weight = p->row_weight;
    g.mn_lbo = 8192;
    g.mn_sbo = 1024;
#ifdef MOMOE_DEBUG_KNOBS
    if (const char* s = getenv("MOMOE_DEBUG_MN_DESC")) {
        unsigned a = 0, b = 0;
        if (sscanf(s, "%u,%u", &a, &b) == 2) { g.mn_lbo = a; g.mn_sbo = b; }
    }
#endif
}

template <int MODE>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& g, cudaStream_t stream) {
    using C = Cfg<MODE>;
    // per-device attribute; setting it on every launch costs well under a microsecond of host time
    if (cudaFuncSetAttribute(grouped_gemm_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::SMEM_BYTES) != cudaSuccess)
        return MOMOE_ERR_CUDA;
    const int grid = sm_count();
    grouped_gemm_kernel<MODE><<<grid, 192, C::SMEM_BYTES, stream>>>(tmA, tmB, g);
    return cudaGetLastError() == cudaSuccess ? MOMOE_OK : MOMOE_ERR_CUDA;
}

static inline int cdiv(int a, int b) { return (a + b - 1) / b; }

}  // namespace momoe

using namespace momoe;

extern "C" __attribute__((visibility("default"))) int momoe_up_swiglu(const momoe_plan_t* plan, const void* x_sorted, const void* W1_ND2H, void* h_sorted,
                               void* a_out, void* b_out, int32_t ab_mode, momoe_stream_t stream) {
    int rc = check_plan(plan);
    if (rc != MOMOE_OK) return rc;
    if (x_sorted == nullptr || W1_ND2H == nullptr) return MOMOE_ERR_ARG;
    if (ab_mode < 0 || ab_mode > 2) return MOMOE_ERR_ARG;
    if (ab_mode != 2 && h_sorted == nullptr) return MOMOE_ERR_ARG;
    if (ab_mode != 0 && (a_out == nullptr || b_out == nullptr)) return MOMOE_ERR_ARG;
    const int D = plan->D, H = plan->H;
    CUtensorMap tmA, tmB;
    if ((rc = encode_tmap_2d(&tmA, x_sorted, plan->rows_capacity, D, TILE_M, TILE_K)) != MOMOE_OK) return rc;
    if ((rc = encode_tmap_3d(&tmB, W1_ND2H, plan->N, D, 2 * H, TILE_K, 64)) != MOMOE_OK) return rc;
    GemmArgs g;
    base_args(plan, g);
    g.n_nblk = cdiv(H, 128);
    g.nkb = cdiv(D, TILE_K);
    g.out_cols = H;
    g.half = H;
    g.ab_mode = ab_mode;
    g.out0 = static_cast<__nv_bfloat16*>(h_sorted);
    g.out1 = static_cast<__nv_bfloat16*>(a_out);
    g.out2 = static_cast<__nv_bfloat16*>(b_out);
    return launch<MODE_UP>(tmA, tmB, g, static_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) int momoe_down_scale(const momoe_plan_t* plan, const void* h_sorted, const void* W2_NHD, void* y_sorted,
                                momoe_stream_t stream) {
    int rc = check_plan(plan);
    if (rc != MOMOE_OK) return rc;
    if (h_sorted == nullptr || W2_NHD == nullptr || y_sorted == nullptr) return MOMOE_ERR_ARG;
    const int D = plan->D, H = plan->H;
    CUtensorMap tmA, tmB;
    if ((rc = encode_tmap_2d(&tmA, h_sorted, plan->rows_capacity, H, TILE_M, TILE_K)) != MOMOE_OK) return rc;
    if ((rc = encode_tmap_3d(&tmB, W2_NHD, plan->N, H, D, TILE_K, 64)) != MOMOE_OK) return rc;
    GemmArgs g;
    base_args(plan, g);
    g.n_nblk = cdiv(D, 256);
    g.nkb = cdiv(H, TILE_K);
    g.out_cols = D;
    g.out0 = static_cast<__nv_bfloat16*>(y_sorted);
    return launch<MODE_DOWN>(tmA, tmB, g, static_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) int momoe_dgrad2_swiglu_bwd(const momoe_plan_t* plan, const void* g_sorted, const void* W2_NHD,
                                       const void* a_saved, const void* b_saved, const void* a_recomp,
                                       const void* b_recomp, void* gz_sorted, void* hs_sorted, float* gs_part,
                                       momoe_stream_t stream) {
    int rc = check_plan(plan);
    if (rc != MOMOE_OK) return rc;
    if (g_sorted == nullptr || W2_NHD == nullptr || gz_sorted == nullptr || hs_sorted == nullptr || gs_part == nullptr)
        return MOMOE_ERR_ARG;
    if ((a_saved == nullptr) != (b_saved == nullptr) || (a_recomp == nullptr) != (b_recomp == nullptr))
        return MOMOE_ERR_ARG;
    if (a_saved == nullptr && a_recomp == nullptr) return MOMOE_ERR_ARG;
    const int D = plan->D, H = plan->H;
    CUtensorMap tmA, tmB;
    if ((rc = encode_tmap_2d(&tmA, g_sorted, plan->rows_capacity, D, TILE_M, TILE_K)) != MOMOE_OK) return rc;
    // W2[e] is [H, D]: as the B operand its rows are the H output columns and D is the contiguous k axis
    if ((rc = encode_tmap_3d(&tmB, W2_NHD, plan->N, H, D, 128, TILE_K)) != MOMOE_OK) return rc;
    GemmArgs g;
    base_args(plan, g);
    g.n_nblk = cdiv(H, 128);
    g.nkb = cdiv(D, TILE_K);
    g.out_cols = H;
    g.out0 = static_cast<__nv_bfloat16*>(gz_sorted);
    g.out1 = static_cast<__nv_bfloat16*>(hs_sorted);
    g.a_saved = static_cast<const __nv_bfloat16*>(a_saved);
    g.b_saved = static_cast<const __nv_bfloat16*>(b_saved);
    g.a_recomp = static_cast<const __nv_bfloat16*>(a_recomp);
    g.b_recomp = static_cast<const __nv_bfloat16*>(b_recomp);
    g.gs_part = gs_part;
    return launch<MODE_DGRAD2>(tmA, tmB, g, static_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) int momoe_dgrad1(const momoe_plan_t* plan, const void* gz_sorted, const void* W1_ND2H, void* gx_sorted,
                            momoe_stream_t stream) {
    int rc = check_plan(plan);
    if (rc != MOMOE_OK) return rc;
    if (gz_sorted == nullptr || W1_ND2H == nullptr || gx_sorted == nullptr) return MOMOE_ERR_ARG;
    const int D = plan->D, H = plan->H;
    CUtensorMap tmA, tmB;
    if ((rc = encode_tmap_2d(&tmA, gz_sorted, plan->rows_capacity, 2 * H, TILE_M, TILE_K)) != MOMOE_OK) return rc;
    // W1[e] is [D, 2H]: rows are the D output columns, 2H is the contiguous k axis
    if ((rc = encode_tmap_3d(&tmB, W1_ND2H, plan->N, D, 2 * H, 256, TILE_K)) != MOMOE_OK) return rc;
    GemmArgs g;
    base_args(plan, g);
    g.n_nblk = cdiv(D, 256);
    g.nkb = cdiv(2 * H, TILE_K);
    g.out_cols = D;
    g.out0 = static_cast<__nv_bfloat16*>(gx_sorted);
    return launch<MODE_DGRAD1>(tmA, tmB, g, static_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) int momoe_wgrad(const momoe_plan_t* plan, const void* a_sorted, int32_t X, const void* b_sorted, int32_t Y,
                           void* dW_NXY, momoe_stream_t stream) {
    int rc = check_plan(plan);
    if (rc != MOMOE_OK) return rc;
    if (a_sorted == nullptr || b_sorted == nullptr || dW_NXY == nullptr || X <= 0 || Y <= 0) return MOMOE_ERR_ARG;
    if (X % 8 != 0 || Y % 8 != 0) return MOMOE_ERR_UNSUPPORTED;
    CUtensorMap tmA, tmB;
    // both operands are read as [64 rows (k) x 64 columns (m or n)] boxes: MN-major
    if ((rc = encode_tmap_2d(&tmA, a_sorted, plan->rows_capacity, X, TILE_K, 64)) != MOMOE_OK) return rc;
    if ((rc = encode_tmap_2d(&tmB, b_sorted, plan->rows_capacity, Y, TILE_K, 64)) != MOMOE_OK) return rc;
    GemmArgs g;
    base_args(plan, g);
    g.n_mblk = cdiv(X, TILE_M);
    g.n_nblk = cdiv(Y, 256);
    g.out_rows = X;
    g.out_cols = Y;
    g.out0 = static_cast<__nv_bfloat16*>(dW_NXY);
    return launch<MODE_WGRAD>(tmA, tmB, g, static_cast<cudaStream_t>(stream));
}
