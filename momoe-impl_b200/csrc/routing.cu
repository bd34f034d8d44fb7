// Router (softmax + top-k with bias), expert-major permutation, row gather / combine, and the small
// backward helpers.  All of this is HBM-bound integer / byte work: warp-level kernels, 128-bit accesses.
#include <cmath>
#include <cstring>
#include <mutex>

#include "internal.h"
#include "../../include/momoe_b200.h"

namespace momoe {

constexpr int MAX_EXPERTS = 1024;
constexpr int MAX_TOPK = 32;
constexpr int CHUNK_TOKENS = 64;  // tokens one warp ranks in the permutation passes

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Butterfly in the order 16, 8, 4, 2, 1: the order torch's warp softmax uses, so the fp32 sum is identical.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ------------------------------------------------------------------------------------------------ router
// One warp per token.  Element j of the gating group lives in lane j % 32, slot j / 32 (the layout of
// torch's warp softmax), so max / exp / sum are evaluated in the same order and p is bit-identical.
template <int NPL>  // gating elements per lane
__global__ void route_topk_kernel(const __nv_bfloat16* __restrict__ logits, const float* __restrict__ biases, int M,
                                  int N, int K, int Ks, int* __restrict__ topk_idx, float* __restrict__ topk_w,
                                  int* __restrict__ mask_NM, float* __restrict__ s_MN,
                                  float* __restrict__ s_postsoft_MN, float* __restrict__ Ng_M,
                                  float* __restrict__ Ks_M) {
    const int lane = threadIdx.x & 31;
    const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (m >= M) return;
    const int Ng = N - Ks;
    const int Kg = K - Ks;
    const __nv_bfloat16* row = logits + static_cast<size_t>(m) * N;

    float p[NPL];
    float score[NPL];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const int j = lane + i * 32;
        p[i] = (j < Ng) ? __bfloat162float(row[j]) : -INFINITY;
        mx = fmaxf(mx, p[i]);
    }
    mx = warp_max(mx);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        p[i] = expf(p[i] - mx);
        sum += p[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const int j = lane + i * 32;
        p[i] = p[i] / sum;
        score[i] = (j < Ng) ? p[i] + biases[j] : -INFINITY;
    }

    // top-Kg by repeated warp arg-max; equal scores resolve to the lowest expert id
    uint32_t picked = 0;  // bit i: slot i of this lane is selected
    for (int k = 0; k < Kg; ++k) {
        float bv = -INFINITY;
        int bj = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int j = lane + i * 32;
            const bool free_slot = ((picked >> i) & 1u) == 0 && j < Ng;
            if (free_slot && (score[i] > bv || bj == 0x7fffffff)) {  // slots ascend in j, so ties keep the lower j
                bv = score[i];
                bj = j;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oj = __shfl_xor_sync(0xffffffffu, bj, o);
            if (oj != 0x7fffffff && (bj == 0x7fffffff || ov > bv || (ov == bv && oj < bj))) {
                bv = ov;
                bj = oj;
            }
        }
        if (bj != 0x7fffffff && (bj & 31) == lane) picked |= 1u << (bj >> 5);
    }

    // renormalise the selected probabilities (sum in ascending expert id)
    float ng = 0.0f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const uint32_t bal = __ballot_sync(0xffffffffu, (picked >> i) & 1u);
        for (uint32_t b = bal; b != 0; b &= b - 1) {
            const int src = __ffs(b) - 1;
            ng += __shfl_sync(0xffffffffu, p[i], src);
        }
    }

    // shared experts: softmax over the last Ks logits (lane = index inside the group)
    float ps = 0.0f, ks_sum = 0.0f;
    if (Ks > 0) {
        float l = (lane < Ks) ? __bfloat162float(row[Ng + lane]) : -INFINITY;
        const float smx = warp_max(l);
        const float e = expf(l - smx);
        const float ssum = warp_sum(e);
        ps = e / ssum;
        ks_sum = 0.0f;
        for (int j = 0; j < Ks; ++j) ks_sum += __shfl_sync(0xffffffffu, ps, j);
    }

    // compact outputs, ascending expert id
    int base = 0;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const bool sel = (picked >> i) & 1u;
        const uint32_t bal = __ballot_sync(0xffffffffu, sel);
        if (sel) {
            const int slot = base + __popc(bal & ((1u << lane) - 1u));
            topk_idx[static_cast<size_t>(m) * K + slot] = lane + i * 32;
            topk_w[static_cast<size_t>(m) * K + slot] = p[i] / ng;
        }
        base += __popc(bal);
    }
    if (lane < Ks) {
        topk_idx[static_cast<size_t>(m) * K + Kg + lane] = Ng + lane;
        topk_w[static_cast<size_t>(m) * K + Kg + lane] = ps / ks_sum;
    }

    if (s_MN != nullptr) {
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int j = lane + i * 32;
            if (j < Ng) {
                const bool sel = (picked >> i) & 1u;
                s_MN[static_cast<size_t>(m) * N + j] = sel ? p[i] / ng : 0.0f;
                s_postsoft_MN[static_cast<size_t>(m) * N + j] = sel ? p[i] : 0.0f;
                if (sel) mask_NM[static_cast<size_t>(j) * M + m] = 1;
            }
        }
        if (lane < Ks) {
            s_MN[static_cast<size_t>(m) * N + Ng + lane] = ps / ks_sum;
            s_postsoft_MN[static_cast<size_t>(m) * N + Ng + lane] = ps;
            mask_NM[static_cast<size_t>(Ng + lane) * M + m] = 1;
        }
    }
    if (Ng_M != nullptr && lane == 0) {
        Ng_M[m] = ng;
        Ks_M[m] = ks_sum;
    }
}

// Dense mask / weights of an external router -> compact [M,K] form (ascending expert id).
__global__ void topk_from_mask_kernel(const int* __restrict__ mask, long long m_sn, long long m_sm,
                                      const float* __restrict__ s, long long s_sn, long long s_sm, int M, int N, int K,
                                      int* __restrict__ topk_idx, float* __restrict__ topk_w, int* status) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= M) return;
    int cnt = 0;
    for (int e = 0; e < N; ++e) {
        if (mask[e * m_sn + m * m_sm] != 0) {
            if (cnt < K) {
                topk_idx[static_cast<size_t>(m) * K + cnt] = e;
                topk_w[static_cast<size_t>(m) * K + cnt] = s[e * s_sn + m * s_sm];
            }
            ++cnt;
        }
    }
    if (cnt != K) {
        atomicCAS(status, 0, DEV_BAD_TOPK_COUNT);
        for (int k = cnt; k < K; ++k) {  // keep later kernels in bounds: route the missing slots to expert 0 with weight 0
            topk_idx[static_cast<size_t>(m) * K + k] = 0;
            topk_w[static_cast<size_t>(m) * K + k] = 0.0f;
        }
    }
}

// ------------------------------------------------------------------------------------------ permutation
// Pass A: per-chunk histogram.  counts[e*n_chunks + c] = tokens of chunk c routed to expert e.
// One warp per chunk; hist = N ints of shared memory owned by the warp.
__device__ __forceinline__ void perm_count_chunk(const int* __restrict__ topk_idx, int M, int N, int K, int n_chunks,
                                                 int* counts, int* status, int chunk, int* hist, int lane) {
    const int m0 = chunk * CHUNK_TOKENS;
    for (int e = lane; e < N; e += 32) hist[e] = 0;
    __syncwarp();
    for (int t = lane; t < CHUNK_TOKENS; t += 32) {
        const int m = m0 + t;
        if (m < M) {
            for (int k = 0; k < K; ++k) {
                int e = topk_idx[static_cast<size_t>(m) * K + k];
                if (e < 0 || e >= N) { atomicCAS(status, 0, DEV_BAD_EXPERT_ID); e = 0; }
                atomicAdd(&hist[e], 1);
            }
        }
    }
    __syncwarp();
    for (int e = lane; e < N; e += 32) counts[static_cast<size_t>(e) * n_chunks + chunk] = hist[e];
    __syncwarp();
}

__global__ void perm_count_kernel(const int* __restrict__ topk_idx, int M, int N, int K, int n_chunks,
                                  int* __restrict__ counts, int* status) {
    extern __shared__ int sh[];
    const int warps = blockDim.x >> 5;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunk = blockIdx.x * warps + w;
    if (chunk * CHUNK_TOKENS >= M) return;
    perm_count_chunk(topk_idx, M, N, K, n_chunks, counts, status, chunk, sh + w * N, lane);
}

// Pass B (one block of at least N threads): per-expert exclusive scan over chunks (in place), then the expert-level
// tables.  s_cum / s_pad (N+1 ints of shared memory each) keep cumsums / pad_off for a caller that goes on in the
// same block.
__device__ __forceinline__ void perm_scan_block(int* counts, int n_chunks, int M, int N, int K, long long save_rows,
                                                long long* __restrict__ sizes, int* __restrict__ cumsums,
                                                int* __restrict__ pad_off, int* __restrict__ tile_expert,
                                                int* __restrict__ pair_info, int* __restrict__ sched,
                                                int tile_capacity, int* s_cum, int* s_pad) {
    __shared__ int s_cnt[MAX_EXPERTS];
    __shared__ int s_pair[MAX_EXPERTS + 1];   // first pair of each expert (a pair = two consecutive tiles of one expert)
    __shared__ int s_saved;
    const int e = threadIdx.x;
    if (e == 0) s_saved = 0;
    {   // one warp per expert (32 experts in flight): warp-wide exclusive scan over that expert's chunks
        const int lane = threadIdx.x & 31;
        for (int x = threadIdx.x >> 5; x < N; x += blockDim.x >> 5) {
            int running = 0;
            int* row = counts + static_cast<size_t>(x) * n_chunks;
            for (int c0 = 0; c0 < n_chunks; c0 += 32) {
                const int c = c0 + lane;
                const int v = c < n_chunks ? row[c] : 0;
                int incl = v;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += t;
                }
                if (c < n_chunks) row[c] = running + incl - v;
                running += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) {
                s_cnt[x] = running;
                sizes[x] = running;
            }
        }
    }
    __syncthreads();
    if (e == 0) {  // N <= 1024: a serial scan costs about a microsecond
        int c = 0, p = 0, pr = 0;
        for (int i = 0; i < N; ++i) {
            s_cum[i] = c;
            s_pad[i] = p;
            s_pair[i] = pr;
            const int nt = (s_cnt[i] + TILE_M - 1) / TILE_M;
            c += s_cnt[i];
            p += nt * TILE_M;
            pr += (nt + 1) / 2;
        }
        s_cum[N] = c;
        s_pad[N] = p;
        s_pair[N] = pr;
    }
    __syncthreads();
    if (e < N) {
        cumsums[e] = s_cum[e];
        pad_off[e] = s_pad[e];
        const int ntile = (s_pad[e + 1] - s_pad[e]) / TILE_M;
        const int t0 = s_pad[e] / TILE_M;
        for (int t = 0; t < ntile && t0 + t < tile_capacity; ++t) tile_expert[t0 + t] = e;
        // pair j of this expert covers tiles t0+2j and (when it exists) t0+2j+1: first tile * 2 + has-second
        for (int j = 0; 2 * j < ntile && s_pair[e] + j < tile_capacity; ++j)
            pair_info[s_pair[e] + j] = (t0 + 2 * j) * 2 + (2 * j + 1 < ntile ? 1 : 0);
        // tiles of this expert whose last row index (in the unpadded order) is below save_rows
        long long fit = (save_rows - s_cum[e]) / TILE_M;
        if (fit < 0) fit = 0;
        if (fit > ntile) fit = ntile;
        if (fit > 0) atomicAdd(&s_saved, static_cast<int>(fit));
    }
    __syncthreads();
    if (e == 0) {
        cumsums[N] = M * K;  // the reference stores the total here unconditionally
        pad_off[N] = s_pad[N];
        sched[SCHED_N_TILES] = s_pad[N] / TILE_M;
        sched[SCHED_N_SAVED_TILES] = s_saved;
        sched[SCHED_PAD_ROWS] = s_pad[N];
        sched[SCHED_N_PAIRS] = s_pair[N];
        for (int i = 4; i < SCHED_WORDS; ++i) sched[i] = 0;
    }
}

__global__ void perm_scan_kernel(int* __restrict__ counts, int n_chunks, int M, int N, int K, long long save_rows,
                                 long long* __restrict__ sizes, int* __restrict__ cumsums, int* __restrict__ pad_off,
                                 int* __restrict__ tile_expert, int* __restrict__ pair_info, int* __restrict__ sched,
                                 int tile_capacity) {
    __shared__ int s_cum[MAX_EXPERTS + 1];
    __shared__ int s_pad[MAX_EXPERTS + 1];
    perm_scan_block(counts, n_chunks, M, N, K, save_rows, sizes, cumsums, pad_off, tile_expert, pair_info, sched,
                    tile_capacity, s_cum, s_pad);
}

// Pass C: every (token, k) pair gets its row.  Inside an expert rows ascend with the token id: a warp walks its
// chunk 32 tokens at a time and ranks the lanes that chose the same expert with a per-expert bit mask.
__device__ __forceinline__ void perm_fill_chunk(const int* __restrict__ topk_idx, const float* __restrict__ topk_w,
                                                const int* chunk_off, const int* cumsums, const int* pad_off, int M,
                                                int N, int K, int n_chunks, int* __restrict__ idx,
                                                int* __restrict__ which, int* __restrict__ row_token,
                                                float* __restrict__ row_weight, int* __restrict__ pos, int chunk,
                                                unsigned* bits, int* running, int lane) {
    const int m0 = chunk * CHUNK_TOKENS;
    for (int e = lane; e < N; e += 32) running[e] = chunk_off[static_cast<size_t>(e) * n_chunks + chunk];
    for (int g0 = 0; g0 < CHUNK_TOKENS; g0 += 32) {
        for (int e = lane; e < N; e += 32) bits[e] = 0u;
        __syncwarp();
        const int m = m0 + g0 + lane;
        const bool live = m < M;
        if (live)
            for (int k = 0; k < K; ++k) {
                int e = topk_idx[static_cast<size_t>(m) * K + k];
                if (e < 0 || e >= N) e = 0;
                atomicOr(&bits[e], 1u << lane);
            }
        __syncwarp();
        if (live)
            for (int k = 0; k < K; ++k) {
                int e = topk_idx[static_cast<size_t>(m) * K + k];
                if (e < 0 || e >= N) e = 0;
                const int rank = running[e] + __popc(bits[e] & ((1u << lane) - 1u));
                const int r = cumsums[e] + rank;
                const int pr = pad_off[e] + rank;
                idx[r] = m;
                which[r] = k;
                row_token[pr] = m;
                row_weight[pr] = topk_w[static_cast<size_t>(m) * K + k];
                pos[static_cast<size_t>(m) * K + k] = pr;
            }
        __syncwarp();
        for (int e = lane; e < N; e += 32) running[e] += __popc(bits[e]);
        __syncwarp();
    }
}

__global__ void perm_fill_kernel(const int* __restrict__ topk_idx, const float* __restrict__ topk_w,
                                 const int* __restrict__ chunk_off, const int* __restrict__ cumsums,
                                 const int* __restrict__ pad_off, int M, int N, int K, int n_chunks,
                                 int* __restrict__ idx,
                                 int* __restrict__ which, int* __restrict__ row_token, float* __restrict__ row_weight,
                                 int* __restrict__ pos) {
    extern __shared__ int sh[];
    const int warps = blockDim.x >> 5;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunk = blockIdx.x * warps + w;
    if (chunk * CHUNK_TOKENS >= M) return;
    perm_fill_chunk(topk_idx, topk_w, chunk_off, cumsums, pad_off, M, N, K, n_chunks, idx, which, row_token,
                    row_weight, pos, chunk, reinterpret_cast<unsigned*>(sh) + w * 2 * N, sh + w * 2 * N + N, lane);
}

// Small batches (a few chunks): the three passes and the initialisation of the padding rows in ONE thread block, so
// that a forward pass of a handful of tokens is not a chain of five dependent launches.  Dynamic shared memory:
// counts [N * n_chunks] followed by 2N ints of scratch for each of the SMALL_WARPS warps that walk chunks.
constexpr int SMALL_WARPS = 16;
constexpr int SMALL_MAX_TOKENS = SMALL_WARPS * CHUNK_TOKENS;   // one chunk per warp
constexpr int SMALL_MAX_EXPERTS = 256;
__global__ void __launch_bounds__(MAX_EXPERTS)
perm_small_kernel(const int* __restrict__ topk_idx, const float* __restrict__ topk_w, int M, int N, int K,
                  int n_chunks, long long save_rows, long long* __restrict__ sizes, int* __restrict__ cumsums,
                  int* __restrict__ idx, int* __restrict__ which, int* __restrict__ pad_off,
                  int* __restrict__ tile_expert, int* __restrict__ pair_info, int* __restrict__ sched,
                  int* __restrict__ row_token, float* __restrict__ row_weight, int* __restrict__ pos,
                  int rows_capacity, int tile_capacity, int* status) {
    extern __shared__ int sh[];
    __shared__ int s_cum[MAX_EXPERTS + 1];
    __shared__ int s_pad[MAX_EXPERTS + 1];
    int* counts = sh;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int* scratch = sh + N * n_chunks + (w < SMALL_WARPS ? w : 0) * 2 * N;
    for (int r = threadIdx.x; r < rows_capacity; r += blockDim.x) {   // padding rows: token -1, weight 0
        row_token[r] = -1;
        row_weight[r] = 0.0f;
    }
    if (w < SMALL_WARPS)
        for (int chunk = w; chunk < n_chunks; chunk += SMALL_WARPS)
            perm_count_chunk(topk_idx, M, N, K, n_chunks, counts, status, chunk, scratch, lane);
    __syncthreads();
    perm_scan_block(counts, n_chunks, M, N, K, save_rows, sizes, cumsums, pad_off, tile_expert, pair_info, sched,
                    tile_capacity, s_cum, s_pad);
    __syncthreads();   // also orders the initialisation of row_token / row_weight before the real rows are written
    if (w < SMALL_WARPS)
        for (int chunk = w; chunk < n_chunks; chunk += SMALL_WARPS)
            perm_fill_chunk(topk_idx, topk_w, counts, s_cum, s_pad, M, N, K, n_chunks, idx, which, row_token,
                            row_weight, pos, chunk, reinterpret_cast<unsigned*>(scratch), scratch + N, lane);
}

// ------------------------------------------------------------------------------------------ row movement
// dst[r,:] = src[row_token[r],:], zeros on padding rows.  Rows whose pitch is a multiple of 32 bytes move in 256-bit
// pieces, four per lane in flight (a 4 KiB row is one batch of loads, then K batches of stores).
struct Vec256 {
    uint32_t v[8];
};
__device__ __forceinline__ Vec256 ld256_nc(const void* p) {
    Vec256 r;
    // every source row is read exactly once
    asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]),
                   "=r"(r.v[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ void st256(void* p, const Vec256& r) {
    asm volatile("st.global.L1::no_allocate.L2::evict_first.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p),
                 "r"(r.v[0]), "r"(r.v[1]), "r"(r.v[2]), "r"(r.v[3]), "r"(r.v[4]), "r"(r.v[5]), "r"(r.v[6]), "r"(r.v[7])
                 : "memory");
}
// Token-major: one warp reads a token's row ONCE and stores it to the K padded rows of the token's experts
// (pos_MK), so the source crosses L2 once instead of K times; afterwards the padding rows are zeroed.
__global__ void gather_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ pos_MK,
                                   const int* __restrict__ row_token, const int* __restrict__ sched, int M, int K,
                                   int vec_per_row, uint4* __restrict__ dst, bool wide) {
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int n32 = vec_per_row >> 1;   // 32-byte pieces per row
    for (int m = wid; m < M; m += warps_total) {
        const uint4* s = src + static_cast<size_t>(m) * vec_per_row;
        const int* pos = pos_MK + static_cast<size_t>(m) * K;
        if (wide) {
            for (int c0 = lane; c0 < n32; c0 += 128) {
                Vec256 t[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (c0 + j * 32 < n32) t[j] = ld256_nc(s + 2 * (c0 + j * 32));
                for (int k = 0; k < K; ++k) {
                    uint4* d = dst + static_cast<size_t>(__ldg(pos + k)) * vec_per_row;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (c0 + j * 32 < n32) st256(d + 2 * (c0 + j * 32), t[j]);
                }
            }
        } else {
            for (int c = lane; c < vec_per_row; c += 32) {
                const uint4 v = __ldg(s + c);
                for (int k = 0; k < K; ++k) dst[static_cast<size_t>(__ldg(pos + k)) * vec_per_row + c] = v;
            }
        }
    }
    const int rows = sched[SCHED_PAD_ROWS];
    for (int r = wid; r < rows; r += warps_total) {
        if (row_token[r] >= 0) continue;
        uint4* d = dst + static_cast<size_t>(r) * vec_per_row;
        for (int c = lane; c < vec_per_row; c += 32) d[c] = make_uint4(0, 0, 0, 0);
    }
}

// Row-major form for callers that only have the row table (plan->pos_MK == NULL): one warp per destination row.
__global__ void gather_rows_by_row_kernel(const uint4* __restrict__ src, const int* __restrict__ row_token,
                                          const int* __restrict__ sched, int vec_per_row, uint4* __restrict__ dst) {
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    const int rows = sched[SCHED_PAD_ROWS];
    for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps_total) {
        const int tok = row_token[r];
        uint4* d = dst + static_cast<size_t>(r) * vec_per_row;
        if (tok >= 0) {
            const uint4* s = src + static_cast<size_t>(tok) * vec_per_row;
            for (int c = lane; c < vec_per_row; c += 32) d[c] = __ldg(s + c);
        } else {
            for (int c = lane; c < vec_per_row; c += 32) d[c] = make_uint4(0, 0, 0, 0);
        }
    }
}

__device__ __forceinline__ void acc_bf16x8(const uint4& q, float (&a)[8]) {
    a[0] += __uint_as_float(q.x << 16); a[1] += __uint_as_float(q.x & 0xFFFF0000u);
    a[2] += __uint_as_float(q.y << 16); a[3] += __uint_as_float(q.y & 0xFFFF0000u);
    a[4] += __uint_as_float(q.z << 16); a[5] += __uint_as_float(q.z & 0xFFFF0000u);
    a[6] += __uint_as_float(q.w << 16); a[7] += __uint_as_float(q.w & 0xFFFF0000u);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

// dst[m,:] = bf16(sum_k src[pos[m,k],:]) with fp32 accumulation in ascending k: deterministic, no atomics.
template <int KT>
__global__ void combine_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ pos, int M, int K,
                                    int vec_per_row, uint4* __restrict__ dst) {
    const long long total = static_cast<long long>(M) * vec_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int m = static_cast<int>(i / vec_per_row);
        const int c = static_cast<int>(i - static_cast<long long>(m) * vec_per_row);
        float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (KT > 0) {
            uint4 q[KT > 0 ? KT : 1];
#pragma unroll
            for (int k = 0; k < KT; ++k)
                q[k] = __ldg(src + static_cast<size_t>(pos[static_cast<size_t>(m) * KT + k]) * vec_per_row + c);
#pragma unroll
            for (int k = 0; k < KT; ++k) acc_bf16x8(q[k], a);
        } else {
            for (int k = 0; k < K; ++k)
                acc_bf16x8(__ldg(src + static_cast<size_t>(pos[static_cast<size_t>(m) * K + k]) * vec_per_row + c), a);
        }
        uint4 o;
        o.x = pack2(a[0], a[1]); o.y = pack2(a[2], a[3]); o.z = pack2(a[4], a[5]); o.w = pack2(a[6], a[7]);
        dst[i] = o;
    }
}

// G_s[e, token] = sum of the row's partial sums (dense output pre-zeroed by the caller side of this file).
__global__ void scatter_gs_kernel(const float* __restrict__ gs_part, int n_part, const int* __restrict__ row_token,
                                  const int* __restrict__ tile_expert, const int* __restrict__ sched, int M,
                                  float* __restrict__ G_s) {
    const int rows = sched[SCHED_PAD_ROWS];
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
        const int tok = row_token[r];
        if (tok < 0) continue;
        float s = 0.0f;
        for (int p = 0; p < n_part; ++p) s += gs_part[static_cast<size_t>(r) * n_part + p];
        G_s[static_cast<size_t>(tile_expert[r / TILE_M]) * M + tok] = s;
    }
}

// Router backward, one warp per token (momoe/topk_router.py:11-56 of the reference).
__global__ void router_backward_kernel(const float* __restrict__ G_s, long long g_sn, long long g_sm,
                                       const float* __restrict__ postsoft, const float* __restrict__ s_norm,
                                       const float* __restrict__ Ng_M, const float* __restrict__ Ks_M,
                                       const int* __restrict__ mask_NM, int M, int N, int Ks,
                                       __nv_bfloat16* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (m >= M) return;
    const int Ng = N - Ks;
    const size_t ro = static_cast<size_t>(m) * N;
    // group 0: gating experts [0, Ng) with the selection mask; group 1: shared experts [Ng, N)
    for (int grp = 0; grp < 2; ++grp) {
        const int lo = grp == 0 ? 0 : Ng;
        const int hi = grp == 0 ? Ng : N;
        if (hi == lo) continue;
        float dot = 0.0f;
        for (int j = lo + lane; j < hi; j += 32) {
            const float gsv = G_s[j * g_sn + m * g_sm];
            const float mk = grp == 0 ? static_cast<float>(mask_NM[static_cast<size_t>(j) * M + m]) : 1.0f;
            dot += gsv * s_norm[ro + j] * mk;
        }
        dot = warp_sum(dot);
        const float inv = 1.0f / (grp == 0 ? Ng_M[m] : Ks_M[m]);
        float t = 0.0f;
        for (int j = lo + lane; j < hi; j += 32) t += (G_s[j * g_sn + m * g_sm] - dot) * inv * postsoft[ro + j];
        t = warp_sum(t);
        for (int j = lo + lane; j < hi; j += 32) {
            const float u = (G_s[j * g_sn + m * g_sm] - dot) * inv;
            out[ro + j] = __float2bfloat16_rn(postsoft[ro + j] * (u - t));
        }
    }
}

// Router backward from the per-row partial sums of the experts' backward pass, without any dense [N,M] tensor.
// One warp per token, lane k owns the token's k-th selected expert.  Same formulas as router_backward_kernel; the
// unnormalised probability of a selected expert is its routing weight times the group's normaliser, and every
// unselected expert has a zero gradient because its masked probability is zero (momoe/topk_router.py:11-56).
__global__ void router_backward_compact_kernel(const float* __restrict__ gs_part, int n_part,
                                               const int* __restrict__ pos_MK, const int* __restrict__ topk_idx,
                                               const float* __restrict__ topk_w, const float* __restrict__ Ng_M,
                                               const float* __restrict__ Ks_M, int M, int N, int K, int Ks,
                                               __nv_bfloat16* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (m >= M) return;
    const int Kg = K - Ks;
    __nv_bfloat16* orow = out + static_cast<size_t>(m) * N;
    for (int j = lane; j < N; j += 32) orow[j] = __float2bfloat16_rn(0.0f);
    __syncwarp();
    float g = 0.0f, w = 0.0f;
    int e = 0;
    if (lane < K) {
        const size_t i = static_cast<size_t>(m) * K + lane;
        const size_t r = (pos_MK != nullptr ? static_cast<size_t>(pos_MK[i]) : i) * n_part;
        for (int p = 0; p < n_part; ++p) g += gs_part[r + p];
        w = topk_w[static_cast<size_t>(m) * K + lane];
        e = topk_idx[static_cast<size_t>(m) * K + lane];
    }
    const bool gating = lane < Kg;
    const bool shared = lane >= Kg && lane < K;
    const float dot_g = warp_sum(gating ? g * w : 0.0f);
    const float dot_s = warp_sum(shared ? g * w : 0.0f);
    const float norm = gating ? Ng_M[m] : (shared ? Ks_M[m] : 1.0f);
    const float u = (g - (gating ? dot_g : dot_s)) * (1.0f / norm);
    const float q = w * norm;
    const float t_g = warp_sum(gating ? u * q : 0.0f);
    const float t_s = warp_sum(shared ? u * q : 0.0f);
    if (lane < K) orow[e] = __float2bfloat16_rn(q * (u - (gating ? t_g : t_s)));
}

// Aux-loss-free balancing: b[e] += rate * sign(c_avg - tokens[e]) for the gating experts (shared experts keep -inf).
__global__ void bias_update_kernel(float* __restrict__ biases, const long long* __restrict__ sizes, int n_gating,
                                   float c_avg, float rate) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_gating) return;
    const float d = c_avg - static_cast<float>(sizes[e]);
    const float sg = d > 0.0f ? 1.0f : (d < 0.0f ? -1.0f : 0.0f);
    biases[e] += rate * sg;
}

static inline int cdiv(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }

}  // namespace momoe

using namespace momoe;

#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? MOMOE_OK : MOMOE_ERR_CUDA)

extern "C" __attribute__((visibility("default"))) int momoe_route_topk(const void* logits_MN, const float* biases_N, int32_t M, int32_t N, int32_t K,
                                int32_t Ks, int32_t* topk_idx_MK, float* topk_w_MK, int32_t* mask_NM, float* s_MN,
                                float* s_postsoft_MN, float* Ng_M, float* Ks_M, momoe_stream_t stream) {
    if (logits_MN == nullptr || biases_N == nullptr || topk_idx_MK == nullptr || topk_w_MK == nullptr)
        return MOMOE_ERR_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || Ks < 0 || Ks >= K || K - Ks > N - Ks) return MOMOE_ERR_ARG;
    if (N > MAX_EXPERTS || K > MAX_TOPK || Ks > 32) return MOMOE_ERR_TOO_LARGE;
    const bool dense = mask_NM != nullptr;
    if (dense != (s_MN != nullptr) || dense != (s_postsoft_MN != nullptr)) return MOMOE_ERR_ARG;
    if ((Ng_M != nullptr) != (Ks_M != nullptr) || (dense && Ng_M == nullptr)) return MOMOE_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dense) {
        if (cudaMemsetAsync(mask_NM, 0, sizeof(int32_t) * static_cast<size_t>(N) * M, st) != cudaSuccess)
            return MOMOE_ERR_CUDA;
    }
    const int Ng = N - Ks;
    const int npl = (Ng + 31) / 32;
    const int warps = 8;
    const dim3 grid(cdiv(M, warps)), block(warps * 32);
    const __nv_bfloat16* lg = static_cast<const __nv_bfloat16*>(logits_MN);
#define ROUTE(NPL)                                                                                              \
    route_topk_kernel<NPL><<<grid, block, 0, st>>>(lg, biases_N, M, N, K, Ks, topk_idx_MK, topk_w_MK, mask_NM, \
                                                   s_MN, s_postsoft_MN, Ng_M, Ks_M)
    if (npl <= 1) ROUTE(1);
    else if (npl <= 2) ROUTE(2);
    else if (npl <= 4) ROUTE(4);
    else if (npl <= 8) ROUTE(8);
    else if (npl <= 16) ROUTE(16);
    else ROUTE(32);
#undef ROUTE
    return LAUNCH_OK();
}

extern "C" __attribute__((visibility("default"))) int momoe_topk_from_mask(const int32_t* mask_NM, int64_t mask_stride_n, int64_t mask_stride_m,
                                    const float* s_NM, int64_t s_stride_n, int64_t s_stride_m, int32_t M, int32_t N,
                                    int32_t K, int32_t* topk_idx_MK, float* topk_w_MK, int32_t* status,
                                    momoe_stream_t stream) {
    if (mask_NM == nullptr || s_NM == nullptr || topk_idx_MK == nullptr || topk_w_MK == nullptr || status == nullptr)
        return MOMOE_ERR_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || K > N) return MOMOE_ERR_ARG;
    if (N > MAX_EXPERTS || K > MAX_TOPK) return MOMOE_ERR_TOO_LARGE;
    topk_from_mask_kernel<<<cdiv(M, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        mask_NM, mask_stride_n, mask_stride_m, s_NM, s_stride_n, s_stride_m, M, N, K, topk_idx_MK, topk_w_MK, status);
    return LAUNCH_OK();
}

extern "C" __attribute__((visibility("default"))) size_t momoe_permutation_workspace_bytes(int32_t M, int32_t N, int32_t K) {
    (void)K;
    if (M <= 0 || N <= 0) return 0;
    const size_t chunks = (static_cast<size_t>(M) + CHUNK_TOKENS - 1) / CHUNK_TOKENS;
    return chunks * N * sizeof(int32_t);
}

extern "C" __attribute__((visibility("default"))) int momoe_permutation_launches(int32_t M, int32_t N, int32_t K) {
    (void)K;
    return (M <= SMALL_MAX_TOKENS && N <= SMALL_MAX_EXPERTS) ? 1 : 3;
}

extern "C" __attribute__((visibility("default"))) int momoe_build_permutation(const int32_t* topk_idx_MK, const float* topk_w_MK, int32_t M, int32_t N,
                                       int32_t K, int64_t save_rows, int64_t* sizes_N, int32_t* cumsums_N1,
                                       int32_t* idx_Msum, int32_t* which_Msum, int32_t* pad_off, int32_t* tile_expert,
                                       int32_t* pair_info, int32_t* sched, int32_t* row_token, float* row_weight, int32_t* pos_MK,
                                       int64_t rows_capacity, void* workspace, size_t workspace_bytes, int32_t* status,
                                       momoe_stream_t stream) {
    if (topk_idx_MK == nullptr || topk_w_MK == nullptr || sizes_N == nullptr || cumsums_N1 == nullptr ||
        idx_Msum == nullptr || which_Msum == nullptr || pad_off == nullptr || tile_expert == nullptr || pair_info == nullptr ||
        sched == nullptr || row_token == nullptr || row_weight == nullptr || pos_MK == nullptr ||
        workspace == nullptr || status == nullptr)
        return MOMOE_ERR_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || K > N || save_rows < 0) return MOMOE_ERR_ARG;
    if (N > MAX_EXPERTS || K > MAX_TOPK) return MOMOE_ERR_TOO_LARGE;
    if (static_cast<int64_t>(M) * K > 0x7fffffffLL - static_cast<int64_t>(N) * TILE_M) return MOMOE_ERR_TOO_LARGE;
    if (rows_capacity < momoe_sorted_rows_capacity(M, K, N)) return MOMOE_ERR_ARG;
    if (workspace_bytes < momoe_permutation_workspace_bytes(M, N, K)) return MOMOE_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int* counts = static_cast<int*>(workspace);
    const int n_chunks = cdiv(M, CHUNK_TOKENS);
    if (momoe_permutation_launches(M, N, K) == 1) {
        // one launch: a handful of tokens must not wait for five dependent launches
        const size_t smem = sizeof(int) * (static_cast<size_t>(N) * n_chunks + static_cast<size_t>(SMALL_WARPS) * 2 * N);
        if (cudaFuncSetAttribute(perm_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem)) != cudaSuccess)
            return MOMOE_ERR_CUDA;
        perm_small_kernel<<<1, MAX_EXPERTS, smem, st>>>(
            topk_idx_MK, topk_w_MK, M, N, K, n_chunks, save_rows, reinterpret_cast<long long*>(sizes_N), cumsums_N1,
            idx_Msum, which_Msum, pad_off, tile_expert, pair_info, sched, row_token, row_weight, pos_MK,
            static_cast<int>(rows_capacity), static_cast<int>(momoe_tile_capacity(M, K, N)), status);
        return LAUNCH_OK();
    }
    const int warps = 4;
    const int blocks = cdiv(n_chunks, warps);
    // padding rows: token -1, weight 0
    if (cudaMemsetAsync(row_token, 0xFF, sizeof(int32_t) * static_cast<size_t>(rows_capacity), st) != cudaSuccess ||
        cudaMemsetAsync(row_weight, 0, sizeof(float) * static_cast<size_t>(rows_capacity), st) != cudaSuccess)
        return MOMOE_ERR_CUDA;
    perm_count_kernel<<<blocks, warps * 32, warps * N * sizeof(int), st>>>(topk_idx_MK, M, N, K, static_cast<int>(n_chunks), counts, status);
    perm_scan_kernel<<<1, MAX_EXPERTS, 0, st>>>(counts, n_chunks, M, N, K, save_rows,
                                                reinterpret_cast<long long*>(sizes_N), cumsums_N1, pad_off,
                                                tile_expert, pair_info, sched,
                                                static_cast<int>(momoe_tile_capacity(M, K, N)));
    perm_fill_kernel<<<blocks, warps * 32, warps * 2 * N * sizeof(int), st>>>(
        topk_idx_MK, topk_w_MK, counts, cumsums_N1, pad_off, M, N, K, static_cast<int>(n_chunks), idx_Msum, which_Msum,
        row_token, row_weight, pos_MK);
    return LAUNCH_OK();
}

extern "C" __attribute__((visibility("default"))) int momoe_gather_rows(const momoe_plan_t* plan, const void* src, int32_t cols, void* dst_sorted,
                                 momoe_stream_t stream) {
    if (plan == nullptr || src == nullptr || dst_sorted == nullptr || plan->row_token == nullptr ||
        plan->sched == nullptr)
        return MOMOE_ERR_ARG;
    if (cols <= 0 || cols % 8 != 0) return MOMOE_ERR_UNSUPPORTED;
    if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst_sorted)) & 15) != 0) return MOMOE_ERR_ARG;
    const int blocks = sm_count() * 8;
    // 256-bit moves need every row to start on a 32-byte boundary
    const bool wide = (cols % 16 == 0) &&
                      (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst_sorted)) & 31) == 0);
    if (plan->pos_MK == nullptr)
        gather_rows_by_row_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint4*>(src), plan->row_token, plan->sched, cols / 8, static_cast<uint4*>(dst_sorted));
    else
        gather_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint4*>(src), plan->pos_MK, plan->row_token, plan->sched, plan->M, plan->K, cols / 8,
            static_cast<uint4*>(dst_sorted), wide);
    return LAUNCH_OK();
}

extern "C" __attribute__((visibility("default"))) int momoe_combine_rows(const momoe_plan_t* plan, const void* src_sorted, int32_t cols, void* dst,
                                  momoe_stream_t stream) {
    if (plan == nullptr || src_sorted == nullptr || dst == nullptr || plan->pos_MK == nullptr) return MOMOE_ERR_ARG;
    if (cols <= 0 || cols % 8 != 0) return MOMOE_ERR_UNSUPPORTED;
    if (((reinterpret_cast<uintptr_t>(src_sorted) | reinterpret_cast<uintptr_t>(dst)) & 15) != 0) return MOMOE_ERR_ARG;
    const int vec = cols / 8;
    const long long total = static_cast<long long>(plan->M) * vec;
    int blocks = cdiv(total, 256);
    const int cap = sm_count() * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint4* s = static_cast<const uint4*>(src_sorted);
    uint4* d = static_cast<uint4*>(dst);
    switch (plan->K) {
        case 2: combine_rows_kernel<2><<<blocks, 256, 0, st>>>(s, plan->pos_MK, plan->M, plan->K, vec, d); break;
        case 4: combine_rows_kernel<4><<<blocks, 256, 0, st>>>(s, plan->pos_MK, plan->M, plan->K, vec, d); break;
        case 6: combine_rows_kernel<6><<<blocks, 256, 0, st>>>(s, plan->pos_MK, plan->M, plan->K, vec, d); break;
        case 8: combine_rows_kernel<8><<<blocks, 256, 0, st>>>(s, plan->pos_MK, plan->M, plan->K, vec, d); break;
        default: combine_rows_kernel<0><<<blocks, 256, 0, st>>>(s, plan->pos_MK, plan->M, plan->K, vec, d); break;
    }
    return LAUNCH_OK();
}

extern "C" __attribute__((visibility("default"))) int momoe_scatter_gs(const momoe_plan_t* plan, const float* gs_part, int32_t n_part, float* G_s_NM,
                                momoe_stream_t stream) {
    if (plan == nullptr || gs_part == nullptr || G_s_NM == nullptr || n_part <= 0 || plan->row_token == nullptr ||
        plan->tile_expert == nullptr)
        return MOMOE_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(G_s_NM, 0, sizeof(float) * static_cast<size_t>(plan->N) * plan->M, st) != cudaSuccess)
        return MOMOE_ERR_CUDA;
    scatter_gs_kernel<<<sm_count() * 4, 256, 0, st>>>(gs_part, n_part, plan->row_token, plan->tile_expert, plan->sched,
                                                      plan->M, G_s_NM);
    return LAUNCH_OK();
}

extern "C" __attribute__((visibility("default"))) int momoe_bias_update(float* biases_N, const int64_t* sizes_N,
                                                                         int32_t N, int32_t Ks, float c_avg,
                                                                         float rate, momoe_stream_t stream) {
    if (biases_N == nullptr || sizes_N == nullptr || N <= 0 || Ks < 0 || Ks >= N) return MOMOE_ERR_ARG;
    bias_update_kernel<<<cdiv(N - Ks, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        biases_N, reinterpret_cast<const long long*>(sizes_N), N - Ks, c_avg, rate);
    return LAUNCH_OK();
}

extern "C" __attribute__((visibility("default"))) int momoe_router_backward(const float* G_s, int64_t gs_stride_n, int64_t gs_stride_m,
                                     const float* s_postsoft_MN, const float* s_MN, const float* Ng_M,
                                     const float* Ks_M, const int32_t* mask_NM, int32_t M, int32_t N, int32_t Ks,
                                     void* G_logits_MN, momoe_stream_t stream) {
    if (G_s == nullptr || s_postsoft_MN == nullptr || s_MN == nullptr || Ng_M == nullptr || Ks_M == nullptr ||
        mask_NM == nullptr || G_logits_MN == nullptr)
        return MOMOE_ERR_ARG;
    if (M <= 0 || N <= 0 || Ks < 0 || Ks >= N) return MOMOE_ERR_ARG;
    const int warps = 8;
    router_backward_kernel<<<cdiv(M, warps), warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        G_s, gs_stride_n, gs_stride_m, s_postsoft_MN, s_MN, Ng_M, Ks_M, mask_NM, M, N, Ks,
        static_cast<__nv_bfloat16*>(G_logits_MN));
    return LAUNCH_OK();
}

extern "C" __attribute__((visibility("default"))) int momoe_router_backward_compact(
    const momoe_plan_t* plan, const float* gs_part, int32_t n_part, const int32_t* topk_idx_MK, const float* topk_w_MK,
    const float* Ng_M, const float* Ks_M, int32_t Ks, void* G_logits_MN, momoe_stream_t stream) {
    if (plan == nullptr || gs_part == nullptr || topk_idx_MK == nullptr || topk_w_MK == nullptr || Ng_M == nullptr ||
        Ks_M == nullptr || G_logits_MN == nullptr)
        return MOMOE_ERR_ARG;
    if (n_part <= 0 || Ks < 0 || Ks >= plan->K || plan->M <= 0) return MOMOE_ERR_ARG;
    if (plan->K > 32) return MOMOE_ERR_TOO_LARGE;
    const int warps = 8;
    router_backward_compact_kernel<<<cdiv(plan->M, warps), warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        gs_part, n_part, plan->pos_MK, topk_idx_MK, topk_w_MK, Ng_M, Ks_M, plan->M, plan->N, plan->K, Ks,
        static_cast<__nv_bfloat16*>(G_logits_MN));
    return LAUNCH_OK();
}

// ------------------------------------------------------------------------------------------------------------
// Permutation builder for callers that cannot hand over a scratch buffer.
//
// momoe_build_permutation needs a caller-allocated workspace for the per-chunk histogram.  Some callers have no
// way to obtain one at the moment they route tokens: a serving engine that gave all of HBM to its own pool at
// start-up and must not call cudaMalloc afterwards, a real-time loop that cannot afford the implicit device
// synchronisation of an allocation, or a plug-in that is only ever handed its input and output tensors.  For
// them the histogram lives in a fixed array inside the library image.  The array occupies device memory on every
// GPU that loads the library, from load until the process exits, so it is kept small (1 MiB).
namespace momoe {

constexpr long long kStaticPermScratchInts = 262144;  // 1 MiB of int32: ceil(M/64) * N must not exceed this

// The histogram itself.  On the host this name is only a handle for the runtime: taking its address in host code
// does not give a device pointer (a kernel handed that value would fault, or on systems where the GPU can reach
// host memory, silently use the wrong bytes).  The device address is looked up with cudaGetSymbolAddress below.
static __device__ __align__(256) int g_perm_scratch[kStaticPermScratchInts];

static std::mutex g_perm_scratch_mu;
static int* g_perm_scratch_dev[64] = {nullptr};  // resolved device address, per device ordinal

// Device address of g_perm_scratch on the CURRENT device; resolved once per device.
static int perm_scratch_address(int** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MOMOE_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_perm_scratch_mu);
    if (g_perm_scratch_dev[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_perm_scratch) != cudaSuccess || p == nullptr) return MOMOE_ERR_CUDA;
        g_perm_scratch_dev[dev] = static_cast<int*>(p);
    }
    *out = g_perm_scratch_dev[dev];
    return MOMOE_OK;
}

}  // namespace momoe

extern "C" __attribute__((visibility("default"))) int momoe_build_permutation_static(
    const int32_t* topk_idx_MK, const float* topk_w_MK, int32_t M, int32_t N, int32_t K, int64_t save_rows,
    int64_t* sizes_N, int32_t* cumsums_N1, int32_t* idx_Msum, int32_t* which_Msum, int32_t* pad_off,
    int32_t* tile_expert, int32_t* pair_info, int32_t* sched, int32_t* row_token, float* row_weight, int32_t* pos_MK,
    int64_t rows_capacity, int32_t* status, momoe_stream_t stream) {
    if (topk_idx_MK == nullptr || topk_w_MK == nullptr || sizes_N == nullptr || cumsums_N1 == nullptr ||
        idx_Msum == nullptr || which_Msum == nullptr || pad_off == nullptr || tile_expert == nullptr || pair_info == nullptr ||
        sched == nullptr || row_token == nullptr || row_weight == nullptr || pos_MK == nullptr || status == nullptr)
        return MOMOE_ERR_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || K > N || save_rows < 0) return MOMOE_ERR_ARG;
    if (N > MAX_EXPERTS || K > MAX_TOPK) return MOMOE_ERR_TOO_LARGE;
    if (static_cast<int64_t>(M) * K > 0x7fffffffLL - static_cast<int64_t>(N) * TILE_M) return MOMOE_ERR_TOO_LARGE;
    if (rows_capacity < momoe_sorted_rows_capacity(M, K, N)) return MOMOE_ERR_ARG;
    const long long n_chunks = (static_cast<long long>(M) + CHUNK_TOKENS - 1) / CHUNK_TOKENS;
    if (n_chunks * N > kStaticPermScratchInts) return MOMOE_ERR_TOO_LARGE;  // histogram would not fit the fixed array
    int* counts = nullptr;
    const int rc = perm_scratch_address(&counts);
    if (rc != MOMOE_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int warps = 4;
    const int blocks = cdiv(n_chunks, warps);
    if (cudaMemsetAsync(row_token, 0xFF, sizeof(int32_t) * static_cast<size_t>(rows_capacity), st) != cudaSuccess ||
        cudaMemsetAsync(row_weight, 0, sizeof(float) * static_cast<size_t>(rows_capacity), st) != cudaSuccess)
        return MOMOE_ERR_CUDA;
    // The array still holds the previous call's histogram.  Nothing has to be cleared: the first pass overwrites
    // every entry [chunk, expert] of the part this call uses before the later passes read it.
    perm_count_kernel<<<blocks, warps * 32, warps * N * sizeof(int), st>>>(topk_idx_MK, M, N, K, static_cast<int>(n_chunks), counts, status);
    perm_scan_kernel<<<1, MAX_EXPERTS, 0, st>>>(counts, static_cast<int>(n_chunks), M, N, K, save_rows,
                                                reinterpret_cast<long long*>(sizes_N), cumsums_N1, pad_off,
                                                tile_expert, pair_info, sched,
                                                static_cast<int>(momoe_tile_capacity(M, K, N)));
    perm_fill_kernel<<<blocks, warps * 32, warps * 2 * N * sizeof(int), st>>>(
        topk_idx_MK, topk_w_MK, counts, cumsums_N1, pad_off, M, N, K, static_cast<int>(n_chunks), idx_Msum, which_Msum,
        row_token, row_weight, pos_MK);
    return LAUNCH_OK();
}
