// Persistent grouped GEMM for sm_100a: TMA -> shared-memory ring -> tcgen05.mma over a CTA PAIR (cta_group::2,
// accumulators in TMEM) -> epilogue warps.  One kernel template serves the five GEMMs of the MoMoE layer; they
// differ in operand majorness and epilogue.
//
// Why CTA pairs: with one CTA per 128x256 tile the kernels were bound by the bytes an SM can take in through TMA
// (48 KiB per 64-wide k-block against 512 MMA cycles); loads alone took 70 % of the kernel time.  A pair of CTAs on
// two SMs computes a 256x256 tile: each CTA loads its own 128 rows of A and only HALF of B (32 KiB per k-block),
// one thread of the leader CTA issues M=256 MMAs that read both CTAs' shared memory, and each CTA's TMEM receives
// its 128 rows x 256 columns.  Every TMA load has exactly one destination CTA.
//
// CTA = 320 threads: warp 0 issues TMA loads (one lane; all 32 lanes when an operand's rows are fetched by token id
// with row-gather loads), warp 1 allocates TMEM and (leader CTA, one lane) issues the MMAs, warps 2..9 read
// accumulators out of TMEM, convert them and hand them to TMA stores through a 4 KiB staging area per warp.  A warp may
// only read the 32 TMEM lanes of its quarter (warp_id % 4), so two warps share each quarter and split the tile's
// columns in halves.  Two accumulator buffers in TMEM (2 x 256 columns) let the epilogue of one tile overlap the
// main loop of the next.
//
// Barriers (mbarrier in shared memory):
//   full[s]      leader only; the leader's producer arms it with the bytes of BOTH CTAs, both CTAs' loads credit it
//   empty[s]     one per CTA; the leader's tcgen05.commit arrives on both when the MMAs have read stage s
//   acc_full[b]  one per CTA; commit arrives on both when the tile's last MMA has completed
//   acc_empty[b] leader only; 16 arrivals = 8 epilogue warps of each CTA
// Every wait is bounded (ptx.cuh); a wait that runs out records a code in the caller's status word and every role
// leaves its loop; the CTAs still meet at the final cluster barrier and free TMEM.
//
// Shared-memory operand layouts (all 128-byte swizzled, as written by TMA with SWIZZLE_128B):
//   K-major operand  [128 rows x 64 k]: row r at byte r*128; descriptor SBO = 1024 (8-row group pitch);
//                    one MMA (k = 16) advances the start address by 32 bytes.
//   MN-major operand two [64 k x 64 mn] boxes of 8 KiB: k-row at byte k*128, boxes 8192 bytes apart;
//                    descriptor LBO = 8192 (mn pitch), SBO = 1024 (8-k group pitch); one MMA advances 2048 bytes.
#include <cstring>

#include "internal.h"
#include "ptx.cuh"
#include "../../include/momoe_b200.h"

namespace momoe {

constexpr int EPI_WARPS = 8;
constexpr int CTA_THREADS = 64 + 32 * EPI_WARPS;
constexpr int PAIR_N = 256;                          // tile width of a CTA pair
constexpr int A_BYTES = TILE_M * TILE_K * 2;         // 16 KiB: this CTA's 128 rows x 64 k
constexpr int B_BYTES = (PAIR_N / 2) * TILE_K * 2;   // 16 KiB: this CTA's half of B x 64 k
constexpr int HALF_BYTES = A_BYTES + B_BYTES;        // one 64-wide k slice
// A pipeline stage holds TWO 64-wide k slices (k-block = 128): the barrier hand-shake per stage costs the issuing
// thread about as many cycles as four MMAs take, so each hand-shake has to cover eight of them.
constexpr int KB = 2 * TILE_K;
constexpr int STAGE_BYTES = 2 * HALF_BYTES;
constexpr int STAGES = 3;
constexpr int EPI_WARP_BYTES = 4096;                     // staging area of one epilogue warp (results -> TMA stores)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * EPI_WARP_BYTES + 1024;  // + slack for 1024-byte alignment
constexpr int ACC_BUFS = 2;
constexpr int TMEM_COLS = 512;

enum GemmMode : int { MODE_UP = 0, MODE_DOWN = 1, MODE_DGRAD2 = 2, MODE_DGRAD1 = 3, MODE_WGRAD = 4 };

struct GemmArgs {
    const int* sched;
    const int* tile_expert;
    const int* pair_info;
    const int* pad_off;
    int* status;
    int n_experts;
    int n_nblk;      // column blocks per row pair (row-tile modes) or per output row block (wgrad)
    int n_mblk;      // wgrad: 256-row blocks of one expert's output matrix
    int nkb;         // row-tile modes: k-blocks of 128
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
    // Rows fetched straight from a token-major matrix instead of an expert-major copy: `rows` (the plan's row_token
    // table) gives the token of every padded row, `gather` says which operand is addressed through it (bit 0: A,
    // bit 1: B, wgrad only), `n_tokens` bounds the indices.
    const int* rows;
    int gather;
    int n_tokens;
};

template <int MODE>
struct Cfg {
    static constexpr bool A_MN = (MODE == MODE_WGRAD);
    static constexpr bool B_MN = (MODE == MODE_UP || MODE == MODE_DOWN || MODE == MODE_WGRAD);
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
__device__ __forceinline__ float sigmoidf_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

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
// 256-bit global accesses (one full 32-byte sector per thread): half as many load/store instructions, which
// matters because the row-per-thread pattern of the epilogues costs one tag look-up per thread and instruction.
__device__ __forceinline__ void st_global_256(void* p, const uint32_t (&v)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]),
                 "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
__device__ __forceinline__ void ld_global_nc_256(const void* p, uint32_t (&v)[8]) {
    asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "l"(p));
}
// Same as store_row32 for rows whose pitch is a multiple of 32 bytes and a fully valid 32-column chunk.
__device__ __forceinline__ void store_row32_wide(__nv_bfloat16* dst, const float (&v)[32]) {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        uint32_t q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = pack_bf16(v[g * 16 + 2 * j], v[g * 16 + 2 * j + 1]);
        st_global_256(dst + g * 16, q);
    }
}
__device__ __forceinline__ void store_row32_auto(__nv_bfloat16* dst, const float (&v)[32], int ncols_left, bool wide) {
    if (wide && ncols_left >= 32) store_row32_wide(dst, v);
    else store_row32(dst, v, ncols_left);
}
// Work item -> coordinates of THIS CTA.
// Row-tile modes: item = pair * n_nblk + nb; a pair is two consecutive 128-row tiles of one expert (the second may be
// missing when the expert has an odd number of tiles).  Wgrad: item = (e * n_mblk + mb) * n_nblk + nb.
struct Work {
    int tile;    // this CTA's row tile (row-tile modes)
    int e;       // expert
    int mb;      // wgrad: 256-row output block
    int nb;      // column block
    int nkb;     // k-blocks
    int row0;    // wgrad: first padded row of the expert
    bool valid;  // this CTA's half of the pair holds real work
    bool skip;   // up/recompute: every tile of the pair is saved, nothing to do (same answer in both CTAs)
};

template <int MODE>
__device__ __forceinline__ Work decode_work(const GemmArgs& g, int item, uint32_t cta_rank) {
    Work w;
    w.skip = false;
    if constexpr (MODE == MODE_WGRAD) {
        w.nb = item % g.n_nblk;
        const int t = item / g.n_nblk;
        w.mb = t % g.n_mblk;
        w.e = t / g.n_mblk;
        w.tile = 0;
        w.row0 = __ldg(g.pad_off + w.e);
        w.nkb = (__ldg(g.pad_off + w.e + 1) - w.row0) / KB;   // padded rows are a multiple of 128
        w.valid = true;
    } else {
        w.nb = item % g.n_nblk;
        const int info = __ldg(g.pair_info + item / g.n_nblk);
        const int t0 = info >> 1;
        const int has2 = info & 1;
        w.tile = t0 + static_cast<int>(cta_rank);
        w.valid = cta_rank == 0 || has2 != 0;
        w.e = __ldg(g.tile_expert + t0);
        w.mb = 0;
        w.nkb = g.nkb;
        w.row0 = 0;
        if (MODE == MODE_UP && g.ab_mode == 2) w.skip = (t0 + has2) < __ldg(g.sched + SCHED_N_SAVED_TILES);
    }
    return w;
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(CTA_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmO0, const __grid_constant__ CUtensorMap tmO1,
                    const __grid_constant__ CUtensorMap tmO2, const GemmArgs g) {
    using C = Cfg<MODE>;

    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_full[STAGES];
    __shared__ uint64_t bar_empty[STAGES];
    __shared__ uint64_t bar_acc_full[ACC_BUFS];
    __shared__ uint64_t bar_acc_empty[ACC_BUFS];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();
    const bool leader = cta_rank == 0;
    const int cluster_id = blockIdx.x >> 1;
    const int n_clusters = gridDim.x >> 1;
    const uint32_t stage_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

    // ---- work range (device-resident schedule; nothing is read back by the host)
    int total_items;
    if constexpr (MODE == MODE_WGRAD) total_items = g.n_experts * g.n_mblk * g.n_nblk;
    else total_items = __ldg(g.sched + SCHED_N_PAIRS) * g.n_nblk;
    if (total_items <= 0 || cluster_id >= total_items) return;  // both CTAs of the cluster leave together

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int b = 0; b < ACC_BUFS; ++b) {
            mbar_init(smem_u32(&bar_acc_full[b]), 1);
            mbar_init(smem_u32(&bar_acc_empty[b]), 2 * EPI_WARPS);  // one arrival per epilogue warp of both CTAs
        }
        fence_mbar_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        tma_prefetch_desc(&tmO0);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&tmem_slot), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
    volatile int* abortp = &abort_flag;

    if (warp == 0 && g.gather != 0) {
        // ================================================================ TMA producer, rows gathered by token id
        // The whole warp works: lane 0 waits for the stage and issues the tiled loads of the operand that is not
        // gathered; every lane issues the row-gather loads of four rows of the gathered operand per 64-wide slice.
        // Padding rows (token -1) repeat the first row of their 128-row tile, which is always a real row of the same
        // expert: every consumer multiplies them by a zero routing weight or by the zero padding rows of the other
        // operand.
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const uint32_t full0 = mapa_shared(smem_u32(&bar_full[0]), 0);   // the leader's barriers
        const int r = static_cast<int>(cta_rank);
        const unsigned n_tok = static_cast<unsigned>(g.n_tokens);
        auto fix = [&](int4& t, int first) {
            t.x = static_cast<unsigned>(t.x) < n_tok ? t.x : first;
            t.y = static_cast<unsigned>(t.y) < n_tok ? t.y : first;
            t.z = static_cast<unsigned>(t.z) < n_tok ? t.z : first;
            t.w = static_cast<unsigned>(t.w) < n_tok ? t.w : first;
        };
        for (int item = cluster_id; ok && item < total_items; item += n_clusters) {
            const Work w = decode_work<MODE>(g, item, cta_rank);
            if (w.skip) continue;
            int4 tok = make_int4(0, 0, 0, 0);
            if constexpr (MODE != MODE_WGRAD) {
                // rows 4*lane .. 4*lane+3 of this CTA's tile; a CTA whose half of the pair is missing loads its
                // partner's rows again (its accumulator is never stored)
                const int t_src = w.valid ? w.tile : w.tile - 1;
                tok = __ldg(reinterpret_cast<const int4*>(g.rows + static_cast<size_t>(t_src) * TILE_M) + lane);
                int first = __shfl_sync(0xffffffffu, tok.x, 0);
                first = static_cast<unsigned>(first) < n_tok ? first : 0;
                fix(tok, first);
            }
            for (int kb = 0; kb < w.nkb; ++kb) {
                int4 tk[2];
                if constexpr (MODE == MODE_WGRAD) {
                    // contraction rows of this k-block: lanes l and l+16 fetch the same four rows for the two
                    // 64-column boxes of the slice; the loads are in flight while lane 0 waits for the stage
                    const int rbase = w.row0 + kb * KB;
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        tk[h] = __ldg(reinterpret_cast<const int4*>(g.rows + rbase + h * TILE_K) + (lane & 15));
                    int first = __shfl_sync(0xffffffffu, tk[0].x, 0);
                    first = static_cast<unsigned>(first) < n_tok ? first : 0;
                    fix(tk[0], first);
                    fix(tk[1], first);
                }
                int okw = 1;
                if (lane == 0)
                    okw = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp, g.status, DEV_TIMEOUT_PRODUCER)
                              ? 1 : 0;
                okw = __shfl_sync(0xffffffffu, okw, 0);
                if (okw == 0) { ok = false; break; }
                const uint32_t full = full0 + static_cast<uint32_t>(stage * sizeof(uint64_t));
                if (lane == 0 && leader) mbar_arrive_expect_tx(smem_u32(&bar_full[stage]), 2 * STAGE_BYTES);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t sa = stage_base + stage * STAGE_BYTES + h * HALF_BYTES;
                    const uint32_t sb = sa + A_BYTES;
                    const int k0 = kb * KB + h * TILE_K;
                    if constexpr (MODE == MODE_WGRAD) {
                        const int r0 = w.row0 + k0;
                        const int i = lane >> 4;          // which 64-column box of the slice
                        const uint32_t off = i * 8192 + (lane & 15) * 512;
                        if (g.gather & 1)
                            tma_gather4_pair(sa + off, &tmA, full, w.mb * 256 + r * 128 + i * 64, tk[h].x, tk[h].y,
                                             tk[h].z, tk[h].w);
                        if (g.gather & 2)
                            tma_gather4_pair(sb + off, &tmB, full, w.nb * PAIR_N + r * 128 + i * 64, tk[h].x, tk[h].y,
                                             tk[h].z, tk[h].w);
                        if (lane == 0) {
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                if (!(g.gather & 1))
                                    tma_load_2d_pair(sa + j * 8192, &tmA, full, w.mb * 256 + r * 128 + j * 64, r0);
                                if (!(g.gather & 2))
                                    tma_load_2d_pair(sb + j * 8192, &tmB, full, w.nb * PAIR_N + r * 128 + j * 64, r0);
                            }
                        }
                    } else {
                        tma_gather4_pair(sa + lane * 512, &tmA, full, k0, tok.x, tok.y, tok.z, tok.w);
                        if (lane == 0) {
                            if constexpr (MODE == MODE_UP) {
#pragma unroll
                                for (int i = 0; i < 2; ++i)
                                    tma_load_3d_pair(sb + i * 8192, &tmB, full, r * g.half + w.nb * 128 + i * 64, k0,
                                                     w.e);
                            } else if constexpr (MODE == MODE_DOWN) {
#pragma unroll
                                for (int i = 0; i < 2; ++i)
                                    tma_load_3d_pair(sb + i * 8192, &tmB, full, w.nb * PAIR_N + r * 128 + i * 64, k0,
                                                     w.e);
                            } else {
                                tma_load_3d_pair(sb, &tmB, full, k0, w.nb * PAIR_N + r * 128, w.e);
                            }
                        }
                    }
                }
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 0) {
        // ================================================================ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int item = cluster_id; ok && item < total_items; item += n_clusters) {
                const Work w = decode_work<MODE>(g, item, cta_rank);
                if (w.skip) continue;
                for (int kb = 0; kb < w.nkb; ++kb) {
                    ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp, g.status, DEV_TIMEOUT_PRODUCER);
                    if (!ok) break;
                    if (leader) mbar_arrive_expect_tx(smem_u32(&bar_full[stage]), 2 * STAGE_BYTES);
                    const uint32_t full = mapa_shared(smem_u32(&bar_full[stage]), 0);   // the leader's barrier
                    const int r = static_cast<int>(cta_rank);
                    // two 64-wide k slices; a slice past the end of the k axis is zero-filled by TMA
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t sa = stage_base + stage * STAGE_BYTES + h * HALF_BYTES;
                        const uint32_t sb = sa + A_BYTES;
                        const int k0 = kb * KB + h * TILE_K;
                        if constexpr (MODE == MODE_WGRAD) {
                            const int r0 = w.row0 + k0;
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                tma_load_2d_pair(sa + i * 8192, &tmA, full, w.mb * 256 + r * 128 + i * 64, r0);
                                tma_load_2d_pair(sb + i * 8192, &tmB, full, w.nb * PAIR_N + r * 128 + i * 64, r0);
                            }
                        } else {
                            tma_load_2d_pair(sa, &tmA, full, k0, w.tile * TILE_M);
                            if constexpr (MODE == MODE_UP) {
                                // the leader loads 128 columns of the linear half of W1[e], its peer the matching
                                // 128 columns of the gate half: accumulator columns 0..127 = a, 128..255 = b
#pragma unroll
                                for (int i = 0; i < 2; ++i)
                                    tma_load_3d_pair(sb + i * 8192, &tmB, full, r * g.half + w.nb * 128 + i * 64, k0,
                                                     w.e);
                            } else if constexpr (MODE == MODE_DOWN) {
#pragma unroll
                                for (int i = 0; i < 2; ++i)
                                    tma_load_3d_pair(sb + i * 8192, &tmB, full, w.nb * PAIR_N + r * 128 + i * 64, k0,
                                                     w.e);
                            } else {
                                // K-major weights: rows = output columns, 64 contiguous k per row
                                tma_load_3d_pair(sb, &tmB, full, k0, w.nb * PAIR_N + r * 128, w.e);
                            }
                        }
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc_bf16(2 * TILE_M, PAIR_N, C::A_MN, C::B_MN);
            // Descriptor halves.  High half (constant): SBO = 1024 >> 4, version 1 (bit 46), 128-byte swizzle
            // (bits 61..63).  Low half: start address >> 4 in [0,14), LBO >> 4 in [16,30).  Only the start address
            // changes from MMA to MMA, so the loop below is a handful of 32-bit adds per MMA.
            constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
            constexpr uint32_t a_lbo = C::A_MN ? (8192u >> 4) : 1u;
            constexpr uint32_t b_lbo = C::B_MN ? (8192u >> 4) : 1u;
            constexpr uint32_t a_kstep = C::A_MN ? (2048u >> 4) : (32u >> 4);   // per 16-wide k step
            constexpr uint32_t b_kstep = C::B_MN ? (2048u >> 4) : (32u >> 4);
            const uint32_t a_lo0 = ((stage_base >> 4) & 0x3FFFu) | (a_lbo << 16);
            const uint32_t b_lo0 = (((stage_base + A_BYTES) >> 4) & 0x3FFFu) | (b_lbo << 16);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t a_lo = a_lo0, b_lo = b_lo0;
            int it = 0;
            bool ok = true;
            for (int item = cluster_id; ok && item < total_items; item += n_clusters) {
                const Work w = decode_work<MODE>(g, item, cta_rank);
                if (w.skip) continue;
                const int ab = it & 1;
                const uint32_t aphase = (it >> 1) & 1u;
                ++it;
                ok = mbar_wait(smem_u32(&bar_acc_empty[ab]), aphase ^ 1u, abortp, g.status, DEV_TIMEOUT_MMA);
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + ab * PAIR_N;
                for (int kb = 0; kb < w.nkb; ++kb) {
                    ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abortp, g.status, DEV_TIMEOUT_MMA);
                    if (!ok) break;
                    umma_bf16_pair_lohi(tmem_d, a_lo, desc_hi, b_lo, desc_hi, idesc, kb != 0 ? 1u : 0u);
#pragma unroll
                    for (uint32_t k = 1; k < 2u * TILE_K / UMMA_K; ++k) {
                        const uint32_t off = (k >> 2) * (HALF_BYTES >> 4);   // second 64-wide slice of the stage
                        umma_bf16_pair_lohi(tmem_d, a_lo + off + (k & 3u) * a_kstep, desc_hi,
                                            b_lo + off + (k & 3u) * b_kstep, desc_hi, idesc, 1u);
                    }
                    umma_commit_pair(smem_u32(&bar_empty[stage]), 3);  // frees the stage in both CTAs
                    a_lo += STAGE_BYTES >> 4;
                    b_lo += STAGE_BYTES >> 4;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; a_lo = a_lo0; b_lo = b_lo0; }
                }
                if (!ok) break;
                if (w.nkb > 0) {
                    umma_commit_pair(smem_u32(&bar_acc_full[ab]), 3);
                } else {
                    // nothing to accumulate (expert without tokens): wake both epilogues, they write zeros
                    mbar_arrive(smem_u32(&bar_acc_full[ab]));
                    mbar_arrive_cluster(mapa_shared(smem_u32(&bar_acc_full[ab]), 1));
                }
            }
        }
    } else {
        // ================================================================ epilogue (warps 2..9, both CTAs)
        // Two ways out, chosen per mode by measurement on the headline layer.  Up/gate and dgrad-2 (one accumulator
        // tile per 16 k-blocks, up to three outputs per element) leave through shared memory: a warp converts its
        // 32 rows x 32 (dgrad-2: 16) columns to bf16, writes them into a slot of its 4 KiB staging area in the swizzled
        // layout of the output's tensor map, and one lane hands the slot to a TMA store; tails are clipped by the
        // tensor map; slots rotate, and a slot is rewritten once the store issued from it has finished READING it
        // (dgrad-2: 0.78-0.81 ms with per-thread stores, 0.69-0.71 ms this way).  Down, dgrad-1 and the weight
        // gradients (an accumulator tile every 8 k-blocks) store straight to global memory, one 32-byte piece per
        // thread and row: the staging hop cost them 5-10 %.
        const int q = warp & 3;            // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;     // accumulator row == TMEM lane
        const int half = (warp - 2) >> 2;  // which half of the tile's 32-column chunks this warp handles
        const uint32_t acc_empty_leader = mapa_shared(smem_u32(&bar_acc_empty[0]), 0);
        constexpr int SLOT_BYTES = MODE == MODE_DGRAD2 ? 1024 : 2048;
        constexpr int NSLOTS = EPI_WARP_BYTES / SLOT_BYTES;
        const uint32_t stage_area = stage_base + STAGES * STAGE_BYTES + (warp - 2) * EPI_WARP_BYTES;
        int n_stored = 0;                  // pieces handed to TMA stores so far (lane 0 owns the bulk groups)
        // slot for the next piece, free to write
        auto slot_acquire = [&]() -> uint32_t {
            if (n_stored >= NSLOTS && lane == 0) bulk_wait_read<NSLOTS - 1>();
            __syncwarp();
            return stage_area + (n_stored % NSLOTS) * SLOT_BYTES;
        };
        // 32 columns of this thread's row (16 packed bf16 pairs) into a [32 rows x 64 bytes] slot, 64-byte swizzle:
        // 16-byte chunk j of row r sits at chunk position j ^ ((r >> 1) & 3)
        auto slot_write64 = [&](uint32_t slot, const uint32_t (&p)[16]) {
            const uint32_t base = slot + lane * 64;
            const uint32_t x = (lane >> 1) & 3;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                st_shared_v4(base + ((j ^ x) << 4), p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
        };
        // 16 columns (8 pairs) into a [32 rows x 32 bytes] slot, 32-byte swizzle: chunk j of row r at j ^ ((r >> 2) & 1)
        auto slot_write32 = [&](uint32_t slot, const uint32_t (&p)[8]) {
            const uint32_t base = slot + lane * 32;
            const uint32_t x = (lane >> 2) & 1;
#pragma unroll
            for (int j = 0; j < 2; ++j)
                st_shared_v4(base + ((j ^ x) << 4), p[4 * j], p[4 * j + 1], p[4 * j + 2], p[4 * j + 3]);
        };
        auto slot_store2d = [&](const CUtensorMap* tm, uint32_t slot, int c0, int c1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(tm, slot, c0, c1);
                bulk_commit();
            }
            ++n_stored;
        };
        auto slot_store3d = [&](const CUtensorMap* tm, uint32_t slot, int c0, int c1, int c2) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                tma_store_3d(tm, slot, c0, c1, c2);
                bulk_commit();
            }
            ++n_stored;
        };
        int it = 0;
        bool ok = true;
        for (int item = cluster_id; ok && item < total_items; item += n_clusters) {
            const Work w = decode_work<MODE>(g, item, cta_rank);
            if (w.skip) continue;
            const int ab = it & 1;
            const uint32_t aphase = (it >> 1) & 1u;
            ++it;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ab * PAIR_N;
            const int row0 = w.tile * TILE_M + q * 32;   // first of this warp's 32 output rows (row-tile modes)
            uint32_t r[32];
            if constexpr (MODE == MODE_DGRAD2) {
                // 16 columns at a time.  The saved / recomputed a,b values do not depend on the accumulator: the first
                // piece is fetched while the main loop is still running, each later one while its predecessor is
                // computed.
                constexpr int PIECES = PAIR_N / 16 / (EPI_WARPS / 4);   // 16-column pieces per warp
                const int part = (warp - 2) >> 2;
                const size_t grow = static_cast<size_t>(w.tile) * TILE_M + row;
                const int H = g.out_cols;
                const bool wide = (H % 16) == 0;   // every a,b row starts on a 32-byte boundary
                const int n_saved = __ldg(g.sched + SCHED_N_SAVED_TILES);
                const bool saved = w.tile < n_saved;
                const size_t abrow =
                    (saved ? static_cast<size_t>(w.tile) : static_cast<size_t>(w.tile - n_saved)) * TILE_M + row;
                const __nv_bfloat16* ap = (saved ? g.a_saved : g.a_recomp) + abrow * H;
                const __nv_bfloat16* bp = (saved ? g.b_saved : g.b_recomp) + abrow * H;
                const int p_begin = part * PIECES, p_end = p_begin + PIECES;
                uint32_t na[8], nb[8];
                auto fetch = [&](int pc) {
                    const int col = w.nb * PAIR_N + pc * 16;
                    if (wide && w.valid && col + 16 <= H) {
                        ld_global_nc_256(ap + col, na);
                        ld_global_nc_256(bp + col, nb);
                        return;
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const bool in = w.valid && col + i * 8 < H;
                        const uint4 qa = in ? __ldg(reinterpret_cast<const uint4*>(ap + col + i * 8)) : make_uint4(0, 0, 0, 0);
                        const uint4 qb = in ? __ldg(reinterpret_cast<const uint4*>(bp + col + i * 8)) : make_uint4(0, 0, 0, 0);
                        na[4 * i] = qa.x; na[4 * i + 1] = qa.y; na[4 * i + 2] = qa.z; na[4 * i + 3] = qa.w;
                        nb[4 * i] = qb.x; nb[4 * i + 1] = qb.y; nb[4 * i + 2] = qb.z; nb[4 * i + 3] = qb.w;
                    }
                };
                fetch(p_begin);
                const float wgt = w.valid ? __ldg(g.row_weight + grow) : 0.0f;
                ok = mbar_wait(smem_u32(&bar_acc_full[ab]), aphase, abortp, g.status, DEV_TIMEOUT_EPILOGUE);
                if (!ok) break;
                tc_fence_after();
                if (w.valid) {
                    float gs = 0.0f;
#pragma unroll 1
                    for (int pc = p_begin; pc < p_end; ++pc) {
                        const int col = w.nb * PAIR_N + pc * 16;
                        if (col >= H) break;
                        uint32_t ca[8], cb[8], r16[16];
#pragma unroll
                        for (int i = 0; i < 8; ++i) { ca[i] = na[i]; cb[i] = nb[i]; }
                        if (pc + 1 < p_end) fetch(pc + 1);
                        tmem_ld16(taddr + pc * 16, r16);
                        tmem_ld_wait();
                        uint32_t o1[8], o2[8], o3[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float a0, a1, b0, b1;
                            unpack_bf16(ca[j], a0, a1);
                            unpack_bf16(cb[j], b0, b1);
                            const float g0 = __uint_as_float(r16[2 * j]);
                            const float g1 = __uint_as_float(r16[2 * j + 1]);
                            const float s0 = sigmoidf_fast(b0), s1 = sigmoidf_fast(b1);
                            const float h0 = bf16_round(a0 * b0 * s0), h1 = bf16_round(a1 * b1 * s1);
                            gs = fmaf(g0, h0, gs);
                            gs = fmaf(g1, h1, gs);
                            const float gh0 = wgt * g0, gh1 = wgt * g1;
                            o1[j] = pack_bf16(gh0 * b0 * s0, gh1 * b1 * s1);
                            o2[j] = pack_bf16(gh0 * a0 * s0 * fmaf(b0, 1.0f - s0, 1.0f),
                                              gh1 * a1 * s1 * fmaf(b1, 1.0f - s1, 1.0f));   // gate half
                            o3[j] = pack_bf16(wgt * h0, wgt * h1);
                        }
                        // gz is addressed as [rows, 2, H] so that the linear half is clipped at H
                        uint32_t slot = slot_acquire();
                        slot_write32(slot, o1);
                        slot_store3d(&tmO0, slot, col, 0, row0);
                        slot = slot_acquire();
                        slot_write32(slot, o2);
                        slot_store3d(&tmO0, slot, col, 1, row0);
                        slot = slot_acquire();
                        slot_write32(slot, o3);
                        slot_store2d(&tmO1, slot, col, row0);
                    }
                    g.gs_part[(grow * g.n_nblk + w.nb) * 2 + part] = gs;   // two partial sums per 256-column block
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (leader) mbar_arrive(smem_u32(&bar_acc_empty[ab]));
                    else mbar_arrive_cluster(acc_empty_leader + ab * static_cast<uint32_t>(sizeof(uint64_t)));
                }
                continue;
            }
            ok = mbar_wait(smem_u32(&bar_acc_full[ab]), aphase, abortp, g.status, DEV_TIMEOUT_EPILOGUE);
            if (!ok) break;
            tc_fence_after();
            uint32_t p[16];
            float v[32];
            const bool wide = (g.out_cols % 16) == 0;   // every output row starts on a 32-byte boundary

            if constexpr (MODE == MODE_UP) {
                const int n_saved = __ldg(g.sched + SCHED_N_SAVED_TILES);
                const bool store_ab = (g.ab_mode == 1 && w.tile < n_saved) || (g.ab_mode == 2 && w.tile >= n_saved);
                const int abrow0 = (g.ab_mode == 2 ? w.tile - n_saved : w.tile) * TILE_M + q * 32;
                if (w.valid) {
#pragma unroll 1
                    for (int c = half * 2; c < half * 2 + 2; ++c) {
                        const int col0 = w.nb * 128 + c * 32;
                        if (col0 >= g.out_cols) break;   // uniform across the warp
                        float a[32];
                        tmem_ld32(taddr + c * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) a[i] = __uint_as_float(r[i]);
                        tmem_ld32(taddr + 128 + c * 32, r);
                        tmem_ld_wait();
                        if (store_ab) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) p[i] = pack_bf16(a[2 * i], a[2 * i + 1]);
                            uint32_t slot = slot_acquire();
                            slot_write64(slot, p);
                            slot_store2d(&tmO1, slot, col0, abrow0);
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                p[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                            slot = slot_acquire();
                            slot_write64(slot, p);
                            slot_store2d(&tmO2, slot, col0, abrow0);
                        }
                        if (g.out0 != nullptr) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const float b0 = __uint_as_float(r[2 * i]), b1 = __uint_as_float(r[2 * i + 1]);
                                p[i] = pack_bf16(b0 * sigmoidf_fast(b0) * a[2 * i], b1 * sigmoidf_fast(b1) * a[2 * i + 1]);
                            }
                            const uint32_t slot = slot_acquire();
                            slot_write64(slot, p);
                            slot_store2d(&tmO0, slot, col0, row0);
                        }
                    }
                }
            } else if constexpr (MODE == MODE_DOWN || MODE == MODE_DGRAD1) {
                const size_t grow = static_cast<size_t>(w.tile) * TILE_M + row;
                if (w.valid) {
                    float wgt = 1.0f;
                    if constexpr (MODE == MODE_DOWN) wgt = __ldg(g.row_weight + grow);
#pragma unroll 1
                    for (int c = half * 4; c < half * 4 + 4; ++c) {
                        const int col0 = w.nb * PAIR_N + c * 32;
                        const int left = g.out_cols - col0;
                        if (left <= 0) break;
                        tmem_ld32(taddr + c * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * wgt;
                        store_row32_auto(g.out0 + grow * g.out_cols + col0, v, left, wide);
                    }
                }
            } else if constexpr (MODE == MODE_DGRAD2) {
                // handled below: its operand prefetch starts before the accumulator wait
            } else {  // MODE_WGRAD
                const int orow = w.mb * 256 + static_cast<int>(cta_rank) * TILE_M + row;
                __nv_bfloat16* dst = g.out0 + (static_cast<size_t>(w.e) * g.out_rows + orow) * g.out_cols;
#pragma unroll 1
                for (int c = half * 4; c < half * 4 + 4; ++c) {
                    const int col0 = w.nb * PAIR_N + c * 32;
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
                    if (orow < g.out_rows) store_row32_auto(dst + col0, v, left, wide);
                }
            }
            // hand the accumulator buffer back to the MMA thread of the leader CTA
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(smem_u32(&bar_acc_empty[ab]));
                else mbar_arrive_cluster(acc_empty_leader + ab * static_cast<uint32_t>(sizeof(uint64_t)));
            }
        }
        // the staging area must outlive every store issued from it
        if (lane == 0) bulk_wait_all<0>();
        __syncwarp();
    }

    // ---- teardown: both CTAs meet (the peer's shared memory and TMEM stay alive until the leader's last MMA has
    // been consumed), then the allocating warps free TMEM
    tc_fence_before();
    __syncthreads();
    if (*abortp) {
        // a wait was abandoned: give loads still in flight time to land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
    }
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------- host side
static int check_plan(const momoe_plan_t* p) {
    if (p == nullptr || p->sched == nullptr || p->tile_expert == nullptr || p->pad_off == nullptr ||
        p->row_weight == nullptr || p->status == nullptr || p->pair_info == nullptr)
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
    g.pair_info = p->pair_info;
    g.pad_off = p->pad_off;
    g.status = p->status;
    g.n_experts = p->N;
    g.row_weight = p->row_weight;
}

// Number of CTA pairs that can be resident at once (the two CTAs of a pair sit on neighbouring SMs).
template <int MODE>
static int resident_pairs() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return sm_count() / 2;
    if (cached[dev] == 0) {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(static_cast<unsigned>(sm_count() / 2 * 2));
        cfg.blockDim = dim3(CTA_THREADS);
        cfg.dynamicSmemBytes = SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, grouped_gemm_kernel<MODE>, &cfg) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = sm_count() / 2;
        }
        if (n > sm_count() / 2) n = sm_count() / 2;
        cached[dev] = n;
    }
    return cached[dev];
}

// Tensor maps of the (up to three) outputs of one launch; unused entries alias the first.
struct OutMaps {
    CUtensorMap m[3];
    int n = 0;
};
// Output matrix [rows, cols] written in [32 rows x 32 columns] pieces (64-byte rows, 64-byte swizzle).
static int out_map_2d(OutMaps& o, int i, void* base, uint64_t rows, uint64_t cols) {
    return encode_tmap_2d(&o.m[i], base, rows, cols, 32, 32, TMAP_SWIZZLE_64B);
}

template <int MODE>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const OutMaps& o, const GemmArgs& g,
                  cudaStream_t stream) {
    // the shared-memory attribute is per device and per function: set it the first time a device launches this mode
    static bool attr_set[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return MOMOE_ERR_CUDA;
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        if (cudaFuncSetAttribute(grouped_gemm_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 SMEM_BYTES) != cudaSuccess)
            return MOMOE_ERR_CUDA;
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const int grid = 2 * resident_pairs<MODE>();
    grouped_gemm_kernel<MODE><<<grid, CTA_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, o.m[0], o.m[1], o.m[2], g);
    return cudaGetLastError() == cudaSuccess ? MOMOE_OK : MOMOE_ERR_CUDA;
}

static inline int cdiv(int a, int b) { return (a + b - 1) / b; }

}  // namespace momoe

using namespace momoe;

// A operand of the row-tile modes: an expert-major matrix read in [128 x 64] boxes, or (tokens = true) the
// token-major matrix [plan->M, cols] read four rows at a time through plan->row_token.
static int a_operand(const momoe_plan_t* plan, const void* src, int cols, bool tokens, CUtensorMap* tm, GemmArgs& g) {
    if (!tokens) return encode_tmap_2d(tm, src, plan->rows_capacity, cols, TILE_M, TILE_K);
    // the row table is read four entries (16 bytes) at a time
    if (plan->row_token == nullptr || (reinterpret_cast<uintptr_t>(plan->row_token) & 15) != 0) return MOMOE_ERR_ARG;
    g.rows = plan->row_token;
    g.gather = 1;
    g.n_tokens = plan->M;
    return encode_tmap_2d(tm, src, plan->M, cols, 1, TILE_K);
}

static int up_swiglu_impl(const momoe_plan_t* plan, const void* x, bool tokens, const void* W1_ND2H, void* h_sorted,
                          void* a_out, void* b_out, int32_t ab_mode, momoe_stream_t stream) {
    int rc = check_plan(plan);
    if (rc != MOMOE_OK) return rc;
    if (x == nullptr || W1_ND2H == nullptr) return MOMOE_ERR_ARG;
    if (ab_mode < 0 || ab_mode > 2) return MOMOE_ERR_ARG;
    if (ab_mode != 2 && h_sorted == nullptr) return MOMOE_ERR_ARG;
    if (ab_mode != 0 && (a_out == nullptr || b_out == nullptr)) return MOMOE_ERR_ARG;
    const int D = plan->D, H = plan->H;
    CUtensorMap tmA, tmB;
    GemmArgs g;
    base_args(plan, g);
    if ((rc = a_operand(plan, x, D, tokens, &tmA, g)) != MOMOE_OK) return rc;
    if ((rc = encode_tmap_3d(&tmB, W1_ND2H, plan->N, D, 2 * H, TILE_K, 64)) != MOMOE_OK) return rc;
    g.n_nblk = cdiv(H, 128);
    g.nkb = cdiv(D, KB);
    g.out_cols = H;
    g.half = H;
    g.ab_mode = ab_mode;
    g.out0 = static_cast<__nv_bfloat16*>(h_sorted);
    g.out1 = static_cast<__nv_bfloat16*>(a_out);
    g.out2 = static_cast<__nv_bfloat16*>(b_out);
    OutMaps o;
    o.m[0] = o.m[1] = o.m[2] = tmA;
    if (h_sorted != nullptr && (rc = out_map_2d(o, 0, h_sorted, plan->rows_capacity, H)) != MOMOE_OK) return rc;
    if (ab_mode != 0) {
        // a_out / b_out hold at most rows_capacity rows; the kernel only writes the tiles the mode selects
        if ((rc = out_map_2d(o, 1, a_out, plan->rows_capacity, H)) != MOMOE_OK) return rc;
        if ((rc = out_map_2d(o, 2, b_out, plan->rows_capacity, H)) != MOMOE_OK) return rc;
    }
    return launch<MODE_UP>(tmA, tmB, o, g, static_cast<cudaStream_t>(stream));
}

#define MOMOE_API extern "C" __attribute__((visibility("default")))

MOMOE_API int momoe_up_swiglu(const momoe_plan_t* plan, const void* x_sorted, const void* W1_ND2H, void* h_sorted,
                              void* a_out, void* b_out, int32_t ab_mode, momoe_stream_t stream) {
    return up_swiglu_impl(plan, x_sorted, false, W1_ND2H, h_sorted, a_out, b_out, ab_mode, stream);
}

MOMOE_API int momoe_up_swiglu_tokens(const momoe_plan_t* plan, const void* x_MD, const void* W1_ND2H, void* h_sorted,
                                     void* a_out, void* b_out, int32_t ab_mode, momoe_stream_t stream) {
    return up_swiglu_impl(plan, x_MD, true, W1_ND2H, h_sorted, a_out, b_out, ab_mode, stream);
}

extern "C" __attribute__((visibility("default"))) int momoe_down_scale(const momoe_plan_t* plan, const void* h_sorted,
                                                                      const void* W2_NHD, void* y_sorted,
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
    g.n_nblk = cdiv(D, PAIR_N);
    g.nkb = cdiv(H, KB);
    g.out_cols = D;
    g.out0 = static_cast<__nv_bfloat16*>(y_sorted);
    OutMaps o;
    o.m[0] = o.m[1] = o.m[2] = tmA;   // this mode stores its results directly
    return launch<MODE_DOWN>(tmA, tmB, o, g, static_cast<cudaStream_t>(stream));
}

static int dgrad2_impl(const momoe_plan_t* plan, const void* gy, bool tokens, const void* W2_NHD, const void* a_saved,
                       const void* b_saved, const void* a_recomp, const void* b_recomp, void* gz_sorted,
                       void* hs_sorted, float* gs_part, momoe_stream_t stream) {
    int rc = check_plan(plan);
    if (rc != MOMOE_OK) return rc;
    if (gy == nullptr || W2_NHD == nullptr || gz_sorted == nullptr || hs_sorted == nullptr || gs_part == nullptr)
        return MOMOE_ERR_ARG;
    if ((a_saved == nullptr) != (b_saved == nullptr) || (a_recomp == nullptr) != (b_recomp == nullptr))
        return MOMOE_ERR_ARG;
    if (a_saved == nullptr && a_recomp == nullptr) return MOMOE_ERR_ARG;
    const int D = plan->D, H = plan->H;
    CUtensorMap tmA, tmB;
    GemmArgs g;
    base_args(plan, g);
    if ((rc = a_operand(plan, gy, D, tokens, &tmA, g)) != MOMOE_OK) return rc;
    // W2[e] is [H, D]: as the B operand its rows are the H output columns and D is the contiguous k axis
    if ((rc = encode_tmap_3d(&tmB, W2_NHD, plan->N, H, D, 128, TILE_K)) != MOMOE_OK) return rc;
    g.n_nblk = cdiv(H, PAIR_N);
    g.nkb = cdiv(D, KB);
    g.out_cols = H;
    g.out0 = static_cast<__nv_bfloat16*>(gz_sorted);
    g.out1 = static_cast<__nv_bfloat16*>(hs_sorted);
    g.a_saved = static_cast<const __nv_bfloat16*>(a_saved);
    g.b_saved = static_cast<const __nv_bfloat16*>(b_saved);
    g.a_recomp = static_cast<const __nv_bfloat16*>(a_recomp);
    g.b_recomp = static_cast<const __nv_bfloat16*>(b_recomp);
    g.gs_part = gs_part;
    OutMaps o;
    {
        // gz [rows, 2H] addressed as [rows, 2, H] so that a piece of the linear half is clipped at column H;
        // pieces of 32 rows x 16 columns (32-byte rows, 32-byte swizzle)
        const uint64_t dims[3] = {static_cast<uint64_t>(H), 2, static_cast<uint64_t>(plan->rows_capacity)};
        const uint64_t strides[2] = {static_cast<uint64_t>(H) * 2, static_cast<uint64_t>(H) * 4};
        const uint32_t box[3] = {16, 1, 32};
        if ((rc = encode_tmap(&o.m[0], gz_sorted, 3, dims, strides, box, TMAP_SWIZZLE_32B)) != MOMOE_OK) return rc;
    }
    if ((rc = encode_tmap_2d(&o.m[1], hs_sorted, plan->rows_capacity, H, 32, 16, TMAP_SWIZZLE_32B)) != MOMOE_OK)
        return rc;
    o.m[2] = o.m[1];
    return launch<MODE_DGRAD2>(tmA, tmB, o, g, static_cast<cudaStream_t>(stream));
}

MOMOE_API int momoe_dgrad2_swiglu_bwd(const momoe_plan_t* plan, const void* g_sorted, const void* W2_NHD,
                                      const void* a_saved, const void* b_saved, const void* a_recomp,
                                      const void* b_recomp, void* gz_sorted, void* hs_sorted, float* gs_part,
                                      momoe_stream_t stream) {
    return dgrad2_impl(plan, g_sorted, false, W2_NHD, a_saved, b_saved, a_recomp, b_recomp, gz_sorted, hs_sorted,
                       gs_part, stream);
}

MOMOE_API int momoe_dgrad2_swiglu_bwd_tokens(const momoe_plan_t* plan, const void* g_MD, const void* W2_NHD,
                                             const void* a_saved, const void* b_saved, const void* a_recomp,
                                             const void* b_recomp, void* gz_sorted, void* hs_sorted, float* gs_part,
                                             momoe_stream_t stream) {
    return dgrad2_impl(plan, g_MD, true, W2_NHD, a_saved, b_saved, a_recomp, b_recomp, gz_sorted, hs_sorted, gs_part,
                       stream);
}

extern "C" __attribute__((visibility("default"))) int momoe_dgrad1(const momoe_plan_t* plan, const void* gz_sorted,
                                                                  const void* W1_ND2H, void* gx_sorted,
                                                                  momoe_stream_t stream) {
    int rc = check_plan(plan);
    if (rc != MOMOE_OK) return rc;
    if (gz_sorted == nullptr || W1_ND2H == nullptr || gx_sorted == nullptr) return MOMOE_ERR_ARG;
    const int D = plan->D, H = plan->H;
    CUtensorMap tmA, tmB;
    if ((rc = encode_tmap_2d(&tmA, gz_sorted, plan->rows_capacity, 2 * H, TILE_M, TILE_K)) != MOMOE_OK) return rc;
    // W1[e] is [D, 2H]: rows are the D output columns, 2H is the contiguous k axis
    if ((rc = encode_tmap_3d(&tmB, W1_ND2H, plan->N, D, 2 * H, 128, TILE_K)) != MOMOE_OK) return rc;
    GemmArgs g;
    base_args(plan, g);
    g.n_nblk = cdiv(D, PAIR_N);
    g.nkb = cdiv(2 * H, KB);
    g.out_cols = D;
    g.out0 = static_cast<__nv_bfloat16*>(gx_sorted);
    OutMaps o;
    o.m[0] = o.m[1] = o.m[2] = tmA;   // this mode stores its results directly
    return launch<MODE_DGRAD1>(tmA, tmB, o, g, static_cast<cudaStream_t>(stream));
}

static int wgrad_impl(const momoe_plan_t* plan, const void* a, int32_t X, bool a_tokens, const void* b, int32_t Y,
                      bool b_tokens, void* dW_NXY, momoe_stream_t stream) {
    int rc = check_plan(plan);
    if (rc != MOMOE_OK) return rc;
    if (a == nullptr || b == nullptr || dW_NXY == nullptr || X <= 0 || Y <= 0) return MOMOE_ERR_ARG;
    if (X % 8 != 0 || Y % 8 != 0) return MOMOE_ERR_UNSUPPORTED;
    if ((a_tokens || b_tokens) &&
        (plan->row_token == nullptr || (reinterpret_cast<uintptr_t>(plan->row_token) & 15) != 0))
        return MOMOE_ERR_ARG;
    CUtensorMap tmA, tmB;
    // both operands are read as [64 rows (k) x 64 columns (m or n)] boxes: MN-major; a token-major operand is read
    // four rows at a time ([1 x 64] boxes) through plan->row_token and lands in the same layout
    if ((rc = a_tokens ? encode_tmap_2d(&tmA, a, plan->M, X, 1, 64)
                       : encode_tmap_2d(&tmA, a, plan->rows_capacity, X, TILE_K, 64)) != MOMOE_OK)
        return rc;
    if ((rc = b_tokens ? encode_tmap_2d(&tmB, b, plan->M, Y, 1, 64)
                       : encode_tmap_2d(&tmB, b, plan->rows_capacity, Y, TILE_K, 64)) != MOMOE_OK)
        return rc;
    GemmArgs g;
    base_args(plan, g);
    if (a_tokens || b_tokens) {
        g.rows = plan->row_token;
        g.gather = (a_tokens ? 1 : 0) | (b_tokens ? 2 : 0);
        g.n_tokens = plan->M;
    }
    g.n_mblk = cdiv(X, 256);
    g.n_nblk = cdiv(Y, PAIR_N);
    g.out_rows = X;
    g.out_cols = Y;
    g.out0 = static_cast<__nv_bfloat16*>(dW_NXY);
    OutMaps o;
    o.m[0] = o.m[1] = o.m[2] = tmA;   // this mode stores its results directly
    return launch<MODE_WGRAD>(tmA, tmB, o, g, static_cast<cudaStream_t>(stream));
}

MOMOE_API int momoe_wgrad(const momoe_plan_t* plan, const void* a_sorted, int32_t X, const void* b_sorted, int32_t Y,
                          void* dW_NXY, momoe_stream_t stream) {
    return wgrad_impl(plan, a_sorted, X, false, b_sorted, Y, false, dW_NXY, stream);
}

MOMOE_API int momoe_wgrad_tokens(const momoe_plan_t* plan, const void* a, int32_t X, int32_t a_is_token_major,
                                 const void* b, int32_t Y, int32_t b_is_token_major, void* dW_NXY,
                                 momoe_stream_t stream) {
    return wgrad_impl(plan, a, X, a_is_token_major != 0, b, Y, b_is_token_major != 0, dW_NXY, stream);
}
