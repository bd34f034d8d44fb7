// Forward GEMMs for small token batches (inference / decode), sm_100a.
//
// With a handful of tokens per expert the two forward GEMMs are weight-streaming problems: every touched expert's
// W1 and W2 must cross HBM once, and the 128-row token tiles of the training kernels are almost entirely padding.
// The training kernels then spend their shared memory on padding rows and their MMA time on 256-row tiles, and the
// bytes of weights an SM has in flight (96 KiB) are too few to cover the HBM latency.
//
// Here the operands swap roles: the WEIGHTS are the M side of the MMA (128 weight columns = 128 TMEM lanes) and a
// block of 32 TOKENS is the N side.  A pipeline stage then holds 32 KiB of weights and only 8 KiB of token rows
// (5 stages = 160 KiB of weights in flight per SM), an MMA covers 128 x 32 x 16 and takes 16 cycles, and the
// kernel is bound by HBM alone.
//
//   up   : lanes  0..63 : D[j, t]      = sum_d W1[e][d, j]     * x[t, d]   (a, 64 columns of the linear half)
//          lanes 64..127: D[64 + j, t] = sum_d W1[e][d, H + j] * x[t, d]   (b, the same 64 columns of the gate half)
//          h[t, j] = bf16(b * sigmoid(b) * a); the warps holding b pass it to the warps holding a through shared
//          memory.  64-column items keep the last wave of the persistent grid short.
//   down : D[c, t]   = sum_h W2[e][h, c] * hrow[t, h];  y[t, c] = bf16(D * routing weight of row t), 128 columns
//
// One CTA (192 threads) per SM, persistent over items = (128-row tile, column block); inside an item one pass
// per 32-row token block that contains real rows (real rows are contiguous from the start of a tile, so three
// probes of row_token tell how many blocks there are).  Padding rows of x are zero, so whole blocks are written.
// Warp 0 (one lane) issues TMA loads, warp 1 allocates TMEM and (one lane) issues MMAs, warps 2..5 are the
// epilogue: thread = one weight column, 32 tokens in registers, stores of one token go to 32 consecutive columns.
// Every wait is bounded (ptx.cuh); a wait that runs out records a code in the caller's status word.
//
// Shared-memory layouts (128-byte swizzle, written by TMA):
//   weights, MN-major: per 64-wide k slice two [64 k x 64 columns] boxes of 8 KiB, 8192 bytes apart
//                      (descriptor LBO = 8192, SBO = 1024; one k = 16 step advances 2048 bytes);
//   tokens, K-major:   per slice one [32 rows x 64 k] box of 4 KiB (SBO = 1024; one k = 16 step advances 32 bytes).
#include <cstring>

#include "internal.h"
#include "ptx.cuh"
#include "../../include/momoe_b200.h"

namespace momoe {

constexpr int DEC_THREADS = 192;
constexpr int DEC_NT = 32;                         // tokens per block (MMA N)
constexpr int DEC_W_SLICE = 128 * TILE_K * 2;      // 16 KiB: 128 weight columns x 64 k
constexpr int DEC_X_SLICE = DEC_NT * TILE_K * 2;   // 4 KiB: 32 token rows x 64 k
constexpr int DEC_TMEM_COLS = 64;                  // 2 buffers x 32 columns
constexpr int DEC_SLICE_BYTES = DEC_W_SLICE + DEC_X_SLICE;   // 20 KiB
constexpr int DEC_STAGE_BYTES = 2 * DEC_SLICE_BYTES;         // k-block of 128: 40 KiB
constexpr int DEC_STAGES = 5;
constexpr int DEC_SMEM_BYTES = DEC_STAGES * DEC_STAGE_BYTES + 1024;

struct DecArgs {
    const int* sched;
    const int* tile_expert;
    const int* row_token;
    const float* row_weight;
    int* status;
    int n_cblk;     // column blocks of the output: 64 wide (up) or 128 wide (down)
    int nkb;        // k-blocks of 128
    int out_cols;   // H (up) or D (down)
    int half;       // up: H, first column of the gate half of W1
    __nv_bfloat16* out;
};

struct DecItem {
    int tile, cb, e, n_tb;
};

__device__ __forceinline__ DecItem dec_decode(const DecArgs& g, int item) {
    DecItem w;
    w.tile = item / g.n_cblk;
    w.cb = item - w.tile * g.n_cblk;
    w.e = __ldg(g.tile_expert + w.tile);
    const int* rt = g.row_token + static_cast<size_t>(w.tile) * TILE_M;
    const int r1 = __ldg(rt + DEC_NT), r2 = __ldg(rt + 2 * DEC_NT), r3 = __ldg(rt + 3 * DEC_NT);
    w.n_tb = 1 + (r1 >= 0) + (r2 >= 0) + (r3 >= 0);
    return w;
}

template <bool UP>
__global__ void __launch_bounds__(DEC_THREADS, 1)
decode_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const DecArgs g) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[DEC_STAGES];
    __shared__ uint64_t bar_empty[DEC_STAGES];
    __shared__ float xch[UP ? 2 : 1][UP ? 2 : 1][UP ? DEC_NT * 32 : 1];   // up: [buffer][column group][token][lane]
    __shared__ uint64_t bar_acc_full[2];
    __shared__ uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t stage_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int total_items = __ldg(g.sched + SCHED_N_TILES) * g.n_cblk;
    if (total_items <= 0 || static_cast<int>(blockIdx.x) >= total_items) return;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < DEC_STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_acc_full[b]), 1);
            mbar_init(smem_u32(&bar_acc_empty[b]), 4);   // one arrival per epilogue warp
        }
        fence_mbar_init();
        tma_prefetch_desc(&tmW);
        tma_prefetch_desc(&tmX);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_slot), DEC_TMEM_COLS);
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
                const DecItem w = dec_decode(g, item);
                for (int tb = 0; ok && tb < w.n_tb; ++tb) {
                    const int xrow = w.tile * TILE_M + tb * DEC_NT;
                    for (int kb = 0; kb < g.nkb; ++kb) {
                        ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp, g.status, DEV_TIMEOUT_PRODUCER);
                        if (!ok) break;
                        const uint32_t full = smem_u32(&bar_full[stage]);
                        mbar_arrive_expect_tx(full, DEC_STAGE_BYTES);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint32_t sw = stage_base + stage * DEC_STAGE_BYTES + h * DEC_SLICE_BYTES;
                            const int k0 = kb * 2 * TILE_K + h * TILE_K;
                            if constexpr (UP) {
                                tma_load_3d(sw, &tmW, full, w.cb * 64, k0, w.e);                    // a columns
                                tma_load_3d(sw + 8192, &tmW, full, g.half + w.cb * 64, k0, w.e);    // b columns
                            } else {
                                tma_load_3d(sw, &tmW, full, w.cb * 128, k0, w.e);
                                tma_load_3d(sw + 8192, &tmW, full, w.cb * 128 + 64, k0, w.e);
                            }
                            tma_load_2d(sw + DEC_W_SLICE, &tmX, full, k0, xrow);
                        }
                        if (++stage == DEC_STAGES) { stage = 0; phase ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(128, DEC_NT, /*a_mn_major=*/true, /*b_mn_major=*/false);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
                const DecItem w = dec_decode(g, item);
                for (int tb = 0; ok && tb < w.n_tb; ++tb) {
                    const int ab = it & 1;
                    const uint32_t aphase = (it >> 1) & 1u;
                    ++it;
                    ok = mbar_wait(smem_u32(&bar_acc_empty[ab]), aphase ^ 1u, abortp, g.status, DEV_TIMEOUT_MMA);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + ab * DEC_NT;
                    for (int kb = 0; kb < g.nkb; ++kb) {
                        ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abortp, g.status, DEV_TIMEOUT_MMA);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint32_t sw = stage_base + stage * DEC_STAGE_BYTES + h * DEC_SLICE_BYTES;
                            const uint64_t dw = umma_smem_desc(sw, 8192, 1024);
                            const uint64_t dx = umma_smem_desc(sw + DEC_W_SLICE, 16, 1024);
#pragma unroll
                            for (uint32_t k = 0; k < TILE_K / UMMA_K; ++k)
                                umma_bf16(tmem_d, dw + k * (2048u >> 4), dx + k * (32u >> 4), idesc,
                                          (kb | h | static_cast<int>(k)) != 0 ? 1u : 0u);
                        }
                        umma_commit(smem_u32(&bar_empty[stage]));
                        if (++stage == DEC_STAGES) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    if (g.nkb > 0) umma_commit(smem_u32(&bar_acc_full[ab]));
                    else mbar_arrive(smem_u32(&bar_acc_full[ab]));
                }
            }
        }
    } else {
        // ================================================================ epilogue (warps 2..5)
        const int q = warp & 3;          // TMEM lane quarter this warp may read
        // up: quarters 0,1 hold a (columns 0..63 of the item), quarters 2,3 hold b of the same columns
        const int wcol = UP ? (q & 1) * 32 + lane : q * 32 + lane;
        int it = 0;
        bool ok = true;
        for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
            const DecItem w = dec_decode(g, item);
            const int col = w.cb * (UP ? 64 : 128) + wcol;
            for (int tb = 0; ok && tb < w.n_tb; ++tb) {
                const int ab = it & 1;
                const uint32_t aphase = (it >> 1) & 1u;
                ++it;
                const size_t row0 = static_cast<size_t>(w.tile) * TILE_M + tb * DEC_NT;
                float wgt = 0.0f;
                if constexpr (!UP) wgt = __ldg(g.row_weight + row0 + lane);   // lane t holds the weight of token t
                ok = mbar_wait(smem_u32(&bar_acc_full[ab]), aphase, abortp, g.status, DEV_TIMEOUT_EPILOGUE);
                if (!ok) break;   // the four epilogue warps wait on the same phase: they all leave here together
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * DEC_NT;
                uint32_t r[32];
                tmem_ld32(taddr, r);
                tmem_ld_wait();
                // the accumulator is in registers: hand the buffer back before the rest
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[ab]));
                float v[32];
                if constexpr (UP) {
                    float* xb = &xch[ab][q & 1][0];
                    if (q >= 2) {
#pragma unroll
                        for (int t = 0; t < 32; ++t) xb[t * 32 + lane] = __uint_as_float(r[t]);
                    }
                    // the a-warp and the b-warp of one column group meet; buffer `ab` is written again two passes
                    // later, after the a-warp has arrived at the next meeting, i.e. after it has read this one
                    asm volatile("bar.sync %0, 64;" ::"r"(1 + (q & 1)) : "memory");
                    if (q >= 2) continue;
#pragma unroll
                    for (int t = 0; t < 32; ++t) {
                        const float a = __uint_as_float(r[t]), b = xb[t * 32 + lane];
                        v[t] = b * __fdividef(1.0f, 1.0f + __expf(-b)) * a;
                    }
                } else {
#pragma unroll
                    for (int t = 0; t < 32; ++t)
                        v[t] = __uint_as_float(r[t]) * __shfl_sync(0xffffffffu, wgt, t);
                }
                if (col < g.out_cols) {
                    __nv_bfloat16* dst = g.out + row0 * g.out_cols + col;
#pragma unroll
                    for (int t = 0; t < 32; ++t) dst[static_cast<size_t>(t) * g.out_cols] = __float2bfloat16_rn(v[t]);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abortp) {
        // a wait was abandoned: give loads still in flight time to land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, DEC_TMEM_COLS);
    }
}

template <bool UP>
static int dec_launch(const CUtensorMap& tmW, const CUtensorMap& tmX, const DecArgs& g, cudaStream_t stream) {
    if (cudaFuncSetAttribute(decode_gemm_kernel<UP>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM_BYTES) !=
        cudaSuccess)
        return MOMOE_ERR_CUDA;
    decode_gemm_kernel<UP><<<sm_count(), DEC_THREADS, DEC_SMEM_BYTES, stream>>>(tmW, tmX, g);
    return cudaGetLastError() == cudaSuccess ? MOMOE_OK : MOMOE_ERR_CUDA;
}

static int dec_check_plan(const momoe_plan_t* p) {
    if (p == nullptr || p->sched == nullptr || p->tile_expert == nullptr || p->row_token == nullptr ||
        p->row_weight == nullptr || p->status == nullptr)
        return MOMOE_ERR_ARG;
    if (p->M <= 0 || p->N <= 0 || p->K <= 0 || p->D <= 0 || p->H <= 0 || p->rows_capacity <= 0) return MOMOE_ERR_ARG;
    if (p->D % 8 != 0 || p->H % 8 != 0) return MOMOE_ERR_UNSUPPORTED;
    if (p->rows_capacity % TILE_M != 0) return MOMOE_ERR_ARG;
    return MOMOE_OK;
}

static void dec_base_args(const momoe_plan_t* p, DecArgs& g) {
    memset(&g, 0, sizeof(g));
    g.sched = p->sched;
    g.tile_expert = p->tile_expert;
    g.row_token = p->row_token;
    g.row_weight = p->row_weight;
    g.status = p->status;
}

}  // namespace momoe

using namespace momoe;

extern "C" __attribute__((visibility("default"))) int momoe_up_swiglu_decode(const momoe_plan_t* plan,
                                                                            const void* x_sorted,
                                                                            const void* W1_ND2H, void* h_sorted,
                                                                            momoe_stream_t stream) {
    int rc = dec_check_plan(plan);
    if (rc != MOMOE_OK) return rc;
    if (x_sorted == nullptr || W1_ND2H == nullptr || h_sorted == nullptr) return MOMOE_ERR_ARG;
    const int D = plan->D, H = plan->H;
    CUtensorMap tmW, tmX;
    if ((rc = encode_tmap_3d(&tmW, W1_ND2H, plan->N, D, 2 * H, TILE_K, 64)) != MOMOE_OK) return rc;
    if ((rc = encode_tmap_2d(&tmX, x_sorted, plan->rows_capacity, D, DEC_NT, TILE_K)) != MOMOE_OK) return rc;
    DecArgs g;
    dec_base_args(plan, g);
    g.n_cblk = (H + 63) / 64;
    g.nkb = (D + 2 * TILE_K - 1) / (2 * TILE_K);
    g.out_cols = H;
    g.half = H;
    g.out = static_cast<__nv_bfloat16*>(h_sorted);
    return dec_launch<true>(tmW, tmX, g, static_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) int momoe_down_scale_decode(const momoe_plan_t* plan,
                                                                             const void* h_sorted,
                                                                             const void* W2_NHD, void* y_sorted,
                                                                             momoe_stream_t stream) {
    int rc = dec_check_plan(plan);
    if (rc != MOMOE_OK) return rc;
    if (h_sorted == nullptr || W2_NHD == nullptr || y_sorted == nullptr) return MOMOE_ERR_ARG;
    const int D = plan->D, H = plan->H;
    CUtensorMap tmW, tmX;
    if ((rc = encode_tmap_3d(&tmW, W2_NHD, plan->N, H, D, TILE_K, 64)) != MOMOE_OK) return rc;
    if ((rc = encode_tmap_2d(&tmX, h_sorted, plan->rows_capacity, H, DEC_NT, TILE_K)) != MOMOE_OK) return rc;
    DecArgs g;
    dec_base_args(plan, g);
    g.n_cblk = (D + 127) / 128;
    g.nkb = (H + 2 * TILE_K - 1) / (2 * TILE_K);
    g.out_cols = D;
    g.half = 0;
    g.out = static_cast<__nv_bfloat16*>(y_sorted);
    return dec_launch<false>(tmW, tmX, g, static_cast<cudaStream_t>(stream));
}
