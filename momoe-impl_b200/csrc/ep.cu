// Expert parallelism over peer memory (NVLink / NVSwitch, one process per GPU).
//
// Every rank owns a contiguous block of N/R experts and a set of buffers that all ranks of the node can address
// (symmetric allocations; the caller passes the R base pointers).  One forward pass:
//
//   momoe_ep_publish_counts   my per-expert token counts -> every peer's counts matrix, then a flag hand-shake
//   momoe_ep_plan             from the R x N matrix every rank derives, without the host: the padded expert-major
//                             layout of its own expert block (the tables of momoe_plan_t) and, for every expert of
//                             every rank, the row where its own tokens start inside the owner's layout
//   momoe_ep_dispatch_rows    gather + send fused: token rows are stored straight into the owner's expert-major
//                             buffer (peer stores), so they arrive already sorted and padded; no staging copy
//   momoe_ep_barrier          flag hand-shake between the ranks
//   (local grouped GEMMs on the received rows)
//   momoe_ep_combine_rows     receive + reduce fused: a token's K result rows are loaded from their owners (peer
//                             loads) and summed in fp32
//
// The backward pass reuses the same plan with the upstream gradient.  Nothing here uses multicast or in-switch
// reduction: plain peer loads and stores.  Every wait on a peer's flag is bounded; when it runs out the kernel records
// a code in the status word and returns.
#include <cstdint>

#include "internal.h"
#include "../../include/momoe_b200.h"

namespace momoe {

constexpr int EP_MAX_RANKS = 8;
constexpr long long kFlagWaitCyclesDefault = 4000000000LL;   // about two seconds of SM clocks
// Limit of every wait on a peer's flag, in SM clock cycles; a host-side setting read at launch time
// (momoe_ep_set_wait_limit).  Always finite.
static long long g_flag_wait_cycles = kFlagWaitCyclesDefault;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Thread s < world: tell peer s that this rank reached `epoch`, then wait until peer s has told us the same.
// flags[p] points at rank p's flag array; slot [r] of it is written by rank r only.
__device__ __forceinline__ void flag_handshake(uint32_t* const* flags, int world, int rank, uint32_t epoch,
                                               int* status, long long wait_cycles) {
    __threadfence_system();
    __syncthreads();
    const int s = threadIdx.x;
    if (s < world) {
        st_release_sys(flags[s] + rank, epoch);
        const uint32_t* mine = flags[rank] + s;
        const long long t0 = clock64();
        // epochs only grow; the signed difference tolerates wrap-around
        while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
            if (clock64() - t0 > wait_cycles) {
                atomicCAS(status, 0, DEV_TIMEOUT_PEER);
                break;
            }
            __nanosleep(200);
        }
    }
    __syncthreads();
}

struct PeerPtrs {
    void* p[EP_MAX_RANKS];
};

__global__ void ep_publish_counts_kernel(const long long* __restrict__ sizes_N, int N, PeerPtrs counts, PeerPtrs flags,
                                         int world, int rank, uint32_t epoch, int* status, long long wait_cycles) {
    for (int e = threadIdx.x; e < N; e += blockDim.x) {
        const int v = static_cast<int>(sizes_N[e]);
        for (int p = 0; p < world; ++p) static_cast<int*>(counts.p[p])[rank * N + e] = v;
    }
    flag_handshake(reinterpret_cast<uint32_t* const*>(flags.p), world, rank, epoch, status, wait_cycles);
}

__global__ void ep_barrier_kernel(PeerPtrs flags, int world, int rank, uint32_t epoch, int* status,
                                  long long wait_cycles) {
    flag_handshake(reinterpret_cast<uint32_t* const*>(flags.p), world, rank, epoch, status, wait_cycles);
}

// One block.  counts_RN[s*N + e] = tokens rank s routes to global expert e.
__global__ void ep_plan_kernel(const int* __restrict__ counts_RN, int world, int rank, int N, double save_percent,
                               long long cap_rows, int tile_capacity, int* __restrict__ dst_base,
                               long long* __restrict__ sizes_global, int* __restrict__ local_count,
                               int* __restrict__ pad_off, int* __restrict__ tile_expert, int* __restrict__ pair_info,
                               int* __restrict__ sched, int* status, int split, int* __restrict__ pair_info_part,
                               int* __restrict__ sched_part) {
    __shared__ int s_tot[1024];       // tokens per global expert, all sources
    __shared__ int s_before[1024];    // of those, from ranks below mine
    __shared__ int s_padoff[1024];    // first padded row of the expert inside its owner's layout
    __shared__ int s_rows[EP_MAX_RANKS];   // padded rows of every rank
    __shared__ int s_over;
    const int Nl = N / world;
    const int e = threadIdx.x;
    if (e == 0) s_over = 0;
    if (e < N) {
        int tot = 0, before = 0;
        for (int s = 0; s < world; ++s) {
            const int c = counts_RN[s * N + e];
            if (s < rank) before += c;
            tot += c;
        }
        s_tot[e] = tot;
        s_before[e] = before;
        sizes_global[e] = tot;
    }
    __syncthreads();
    if (e < world) {   // one thread per owner rank: padded offsets of its block
        int p = 0;
        for (int el = 0; el < Nl; ++el) {
            s_padoff[e * Nl + el] = p;
            p += (s_tot[e * Nl + el] + TILE_M - 1) / TILE_M * TILE_M;
        }
        s_rows[e] = p;
        if (p > cap_rows) s_over = 1;
    }
    __syncthreads();
    const bool over = s_over != 0;   // every rank sees the same matrix, so every rank takes the same decision
    if (e < N) dst_base[e] = over ? -1 : s_padoff[e] + s_before[e];
    if (e == 0 && over) atomicCAS(status, 0, DEV_EP_OVERFLOW);
    // this rank's own block
    if (e < Nl) {
        const int ge = rank * Nl + e;
        const int cnt = over ? 0 : s_tot[ge];
        local_count[e] = cnt;
        const int p0 = over ? 0 : s_padoff[ge];
        pad_off[e] = p0;
        const int ntile = (cnt + TILE_M - 1) / TILE_M;
        for (int t = 0; t < ntile && p0 / TILE_M + t < tile_capacity; ++t) tile_expert[p0 / TILE_M + t] = e;
    }
    __syncthreads();
    if (e == 0) {
        // serial pass over the local block: pair table, unpadded prefix for the save rule
        int pairs = 0, unpadded = 0, total = 0;
        int part_pairs[2] = {0, 0}, part_rows[2] = {0, 0};
        for (int el = 0; el < Nl; ++el) total += over ? 0 : s_tot[rank * Nl + el];
        const long long save_rows = static_cast<long long>(static_cast<double>(total) * save_percent / 100.0);
        int saved = 0;
        for (int el = 0; el < Nl; ++el) {
            const int cnt = over ? 0 : s_tot[rank * Nl + el];
            const int ntile = (cnt + TILE_M - 1) / TILE_M;
            const int t0 = (over ? 0 : s_padoff[rank * Nl + el]) / TILE_M;
            for (int j = 0; 2 * j < ntile && pairs < tile_capacity; ++j) {
                const int info = (t0 + 2 * j) * 2 + (2 * j + 1 < ntile ? 1 : 0);
                pair_info[pairs++] = info;
                if (pair_info_part != nullptr) {
                    // the same pair again in the table of its part: local experts below `split`, and the rest
                    const int part = el < split ? 0 : 1;
                    pair_info_part[part * tile_capacity + part_pairs[part]++] = info;
                }
            }
            part_rows[el < split ? 0 : 1] += ntile * TILE_M;
            long long fit = (save_rows - unpadded) / TILE_M;
            if (fit < 0) fit = 0;
            if (fit > ntile) fit = ntile;
            saved += static_cast<int>(fit);
            unpadded += cnt;
        }
        const int rows = over ? 0 : s_rows[rank];
        pad_off[Nl] = rows;
        sched[SCHED_N_TILES] = rows / TILE_M;
        sched[SCHED_N_SAVED_TILES] = saved;
        sched[SCHED_PAD_ROWS] = rows;
        sched[SCHED_N_PAIRS] = pairs;
        for (int i = 4; i < SCHED_WORDS; ++i) sched[i] = 0;
        if (sched_part != nullptr) {
            // tile numbers stay those of the whole block, so the boundary of the saved tiles is the same number
            for (int part = 0; part < 2; ++part) {
                int* sp = sched_part + part * SCHED_WORDS;
                for (int i = 0; i < SCHED_WORDS; ++i) sp[i] = 0;
                sp[SCHED_N_TILES] = rows / TILE_M;
                sp[SCHED_N_SAVED_TILES] = saved;
                sp[SCHED_PAD_ROWS] = part_rows[part];
                sp[SCHED_N_PAIRS] = part_pairs[part];
            }
        }
    }
}

__device__ __forceinline__ void st_256(void* p, const uint4& a, const uint4& b) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
                 "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}

// Gather + send.  One warp per row of this rank's (home) expert-major order.
//   real row pr (token t, expert e, i-th of my tokens for e): src[t,:] -> owner(e)'s rows[dst_base[e] + i, :]
// and, independently, the padding rows of MY OWN receive buffer are zeroed (nobody else writes them).
// Rows are visited round-robin over the destination ranks, starting with the next rank: consecutive warps (and the
// successive rows of one warp) store to different GPUs, so every rank feeds all of its links at once and no GPU is
// the target of all ranks at the same moment (marching through the expert-major order would make every rank send to
// rank 0 first, then to rank 1, ...).
__global__ void __launch_bounds__(256, 4)
ep_dispatch_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ home_row_token,
                        const int* __restrict__ home_tile_expert, const int* __restrict__ home_pad_off,
                        const float* __restrict__ home_row_weight, const int* __restrict__ dst_base, int Nl,
                        int vec_per_row, PeerPtrs rows, PeerPtrs row_w, int* __restrict__ remote_row, int rank,
                        int world, const int* __restrict__ local_count, const int* __restrict__ local_pad_off,
                        bool wide, const int* __restrict__ status, int e_lo, int e_hi) {
    // a hand-shake that timed out leaves counts and plans that cannot be trusted: no payload is sent then; like an
    // overflow (302, dst_base = -1) the rows still get an in-range remote_row so that later reads stay inside the buffers
    const bool no_send = status != nullptr && *reinterpret_cast<const volatile int*>(status) == DEV_TIMEOUT_PEER;
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    // Only rows of the owners' local experts [e_lo, e_hi) are sent: for one destination these are one contiguous run
    // of my expert-major rows.
    int max_len = 0;   // longest of the per-destination runs
    for (int d = 0; d < world; ++d)
        max_len = max(max_len, home_pad_off[d * Nl + e_hi] - home_pad_off[d * Nl + e_lo]);
    const long long n_slots = static_cast<long long>(max_len) * world;
    // a warp changes its destination from one row to the next (a bijection while the warp count is a multiple of the
    // rank count), so that no warp only ever serves the fast local copies
    const bool rotate = warps_total % world == 0;
    for (long long j = wid; j < n_slots; j += warps_total) {
        const int off = static_cast<int>(j / world);
        int d = static_cast<int>(j - static_cast<long long>(off) * world);
        if (rotate) d = static_cast<int>((d + j / warps_total) % world);
        d += rank + 1;
        if (d >= world) d -= world;
        const int lo = home_pad_off[d * Nl + e_lo];
        if (off >= home_pad_off[d * Nl + e_hi] - lo) continue;
        const int pr = lo + off;
        const int tok = home_row_token[pr];
        if (tok < 0) continue;
        const int e = home_tile_expert[pr / TILE_M];
        const int base = no_send ? -1 : dst_base[e];
        if (base < 0) {   // capacity exceeded somewhere, or a peer is missing: nothing is sent (the status word records it)
            if (lane == 0 && remote_row != nullptr) remote_row[pr] = 0;   // keep later reads inside the buffers
            continue;
        }
        const int row = base + (pr - home_pad_off[e]);
        uint4* dst = static_cast<uint4*>(rows.p[d]) + static_cast<size_t>(row) * vec_per_row;
        const uint4* s = src + static_cast<size_t>(tok) * vec_per_row;
        if (wide) {
            // all loads of a batch first, then the (posted) peer stores: four 32-byte pieces per lane in flight
            for (int c0 = lane * 2; c0 < vec_per_row; c0 += 256) {
                uint4 t[8];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (c0 + j * 64 < vec_per_row) {
                        t[2 * j] = __ldg(s + c0 + j * 64);
                        t[2 * j + 1] = __ldg(s + c0 + j * 64 + 1);
                    }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (c0 + j * 64 < vec_per_row) st_256(dst + c0 + j * 64, t[2 * j], t[2 * j + 1]);
            }
        } else {
            for (int c = lane; c < vec_per_row; c += 32) dst[c] = __ldg(s + c);
        }
        if (lane == 0) {
            if (row_w.p[0] != nullptr) static_cast<float*>(row_w.p[d])[row] = home_row_weight[pr];
            if (remote_row != nullptr) remote_row[pr] = row;
        }
    }
    // padding rows of my own receive buffer
    uint4* mine = static_cast<uint4*>(rows.p[rank]);
    float* mine_w = row_w.p[0] != nullptr ? static_cast<float*>(row_w.p[rank]) : nullptr;
    for (int el = e_lo; el < e_hi; ++el) {
        const int lo = local_pad_off[el] + local_count[el];
        const int hi = local_pad_off[el + 1];
        for (int r = lo + wid; r < hi; r += warps_total) {
            uint4* d = mine + static_cast<size_t>(r) * vec_per_row;
            for (int c = lane; c < vec_per_row; c += 32) d[c] = make_uint4(0, 0, 0, 0);
            if (lane == 0 && mine_w != nullptr) mine_w[r] = 0.0f;
        }
    }
}

__device__ __forceinline__ uint4 ld_peer(const uint4* p) {   // bypass L1: the line may have been rewritten by its owner
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void acc8(const uint4& q, float (&a)[8]) {
    a[0] += __uint_as_float(q.x << 16); a[1] += __uint_as_float(q.x & 0xFFFF0000u);
    a[2] += __uint_as_float(q.y << 16); a[3] += __uint_as_float(q.y & 0xFFFF0000u);
    a[4] += __uint_as_float(q.z << 16); a[5] += __uint_as_float(q.z & 0xFFFF0000u);
    a[6] += __uint_as_float(q.w << 16); a[7] += __uint_as_float(q.w & 0xFFFF0000u);
}
__device__ __forceinline__ uint32_t pk(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

// Receive + reduce.  dst[m,:] = bf16(sum_k rows@owner_k[remote_row_k, :]) with fp32 accumulation in ascending k.
template <int KT>
__global__ void ep_combine_rows_kernel(PeerPtrs rows, const int* __restrict__ home_pos,
                                       const int* __restrict__ home_tile_expert, const int* __restrict__ remote_row,
                                       int Nl, int M, int vec_per_row, uint4* __restrict__ dst) {
    const long long total = static_cast<long long>(M) * vec_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int m = static_cast<int>(i / vec_per_row);
        const int c = static_cast<int>(i - static_cast<long long>(m) * vec_per_row);
        uint4 q[KT];
#pragma unroll
        for (int k = 0; k < KT; ++k) {
            const int pr = home_pos[static_cast<size_t>(m) * KT + k];
            const int d = home_tile_expert[pr / TILE_M] / Nl;
            const int row = remote_row[pr];
            q[k] = ld_peer(static_cast<const uint4*>(rows.p[d]) + static_cast<size_t>(row) * vec_per_row + c);
        }
        float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int k = 0; k < KT; ++k) acc8(q[k], a);
        dst[i] = make_uint4(pk(a[0], a[1]), pk(a[2], a[3]), pk(a[4], a[5]), pk(a[6], a[7]));
    }
}
__global__ void ep_combine_rows_generic_kernel(PeerPtrs rows, const int* __restrict__ home_pos,
                                               const int* __restrict__ home_tile_expert,
                                               const int* __restrict__ remote_row, int Nl, int M, int K,
                                               int vec_per_row, uint4* __restrict__ dst) {
    const long long total = static_cast<long long>(M) * vec_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int m = static_cast<int>(i / vec_per_row);
        const int c = static_cast<int>(i - static_cast<long long>(m) * vec_per_row);
        float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int k = 0; k < K; ++k) {
            const int pr = home_pos[static_cast<size_t>(m) * K + k];
            const int d = home_tile_expert[pr / TILE_M] / Nl;
            acc8(ld_peer(static_cast<const uint4*>(rows.p[d]) + static_cast<size_t>(remote_row[pr]) * vec_per_row + c), a);
        }
        dst[i] = make_uint4(pk(a[0], a[1]), pk(a[2], a[3]), pk(a[4], a[5]), pk(a[6], a[7]));
    }
}

// Receive only: the result rows of this rank's (token, expert) pairs whose expert is one of the owners' local experts
// [e_lo, e_hi) are copied from their owners into `staged`, a local buffer indexed like this rank's own expert-major
// order (row pr of `home`).  One warp per row, destinations visited round-robin as in the dispatch.  The sum over a
// token's K rows is left to momoe_ep_combine_rows_staged, which reads these rows from local memory, so the order of
// the fp32 summation does not depend on how the transfer was split.
__global__ void __launch_bounds__(256, 4)
ep_pull_rows_kernel(PeerPtrs rows, const int* __restrict__ home_row_token, const int* __restrict__ home_pad_off,
                    const int* __restrict__ remote_row, int Nl, int vec_per_row, uint4* __restrict__ staged, int rank,
                    int world, int e_lo, int e_hi) {
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int max_len = 0;
    for (int d = 0; d < world; ++d)
        max_len = max(max_len, home_pad_off[d * Nl + e_hi] - home_pad_off[d * Nl + e_lo]);
    const long long n_slots = static_cast<long long>(max_len) * world;
    const bool rotate = warps_total % world == 0;
    for (long long j = wid; j < n_slots; j += warps_total) {
        const int off = static_cast<int>(j / world);
        int d = static_cast<int>(j - static_cast<long long>(off) * world);
        if (rotate) d = static_cast<int>((d + j / warps_total) % world);
        d += rank + 1;
        if (d >= world) d -= world;
        const int lo = home_pad_off[d * Nl + e_lo];
        if (off >= home_pad_off[d * Nl + e_hi] - lo) continue;
        const int pr = lo + off;
        if (home_row_token[pr] < 0) continue;
        const uint4* s = static_cast<const uint4*>(rows.p[d]) + static_cast<size_t>(remote_row[pr]) * vec_per_row;
        uint4* dst = staged + static_cast<size_t>(pr) * vec_per_row;
        for (int c0 = lane; c0 < vec_per_row; c0 += 128) {
            uint4 t[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (c0 + i * 32 < vec_per_row) t[i] = ld_peer(s + c0 + i * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (c0 + i * 32 < vec_per_row) dst[c0 + i * 32] = t[i];
        }
    }
}

// momoe_ep_combine_rows with part of the rows already local: a row whose expert is one of its owner's local experts
// [e_lo, e_hi) is read from `staged` (row pr), every other row from its owner.  Same fp32 summation in ascending k.
template <int KT>
__global__ void ep_combine_rows_staged_kernel(PeerPtrs rows, const int* __restrict__ home_pos,
                                              const int* __restrict__ home_tile_expert,
                                              const int* __restrict__ remote_row, int Nl, int M, int K, int vec_per_row,
                                              uint4* __restrict__ dst, const uint4* __restrict__ staged, int e_lo,
                                              int e_hi) {
    const long long total = static_cast<long long>(M) * vec_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int m = static_cast<int>(i / vec_per_row);
        const int c = static_cast<int>(i - static_cast<long long>(m) * vec_per_row);
        float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (KT > 0) {
            uint4 q[KT > 0 ? KT : 1];
#pragma unroll
            for (int k = 0; k < KT; ++k) {
                const int pr = home_pos[static_cast<size_t>(m) * KT + k];
                const int e = home_tile_expert[pr / TILE_M];
                const int d = e / Nl;
                const int le = e - d * Nl;
                if (le >= e_lo && le < e_hi) q[k] = staged[static_cast<size_t>(pr) * vec_per_row + c];
                else q[k] = ld_peer(static_cast<const uint4*>(rows.p[d]) + static_cast<size_t>(remote_row[pr]) * vec_per_row + c);
            }
#pragma unroll
            for (int k = 0; k < KT; ++k) acc8(q[k], a);
        } else {
            for (int k = 0; k < K; ++k) {
                const int pr = home_pos[static_cast<size_t>(m) * K + k];
                const int e = home_tile_expert[pr / TILE_M];
                const int d = e / Nl;
                const int le = e - d * Nl;
                if (le >= e_lo && le < e_hi) acc8(staged[static_cast<size_t>(pr) * vec_per_row + c], a);
                else acc8(ld_peer(static_cast<const uint4*>(rows.p[d]) + static_cast<size_t>(remote_row[pr]) * vec_per_row + c), a);
            }
        }
        dst[i] = make_uint4(pk(a[0], a[1]), pk(a[2], a[3]), pk(a[4], a[5]), pk(a[6], a[7]));
    }
}

// Per-row dL/ds of the local rows: sum of the partial sums written by the dgrad-2 epilogue.
__global__ void ep_reduce_gs_kernel(const float* __restrict__ gs_part, int n_part, const int* __restrict__ sched,
                                    float* __restrict__ row_gs) {
    const int rows = sched[SCHED_PAD_ROWS];
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
        float s = 0.0f;
        for (int p = 0; p < n_part; ++p) s += gs_part[static_cast<size_t>(r) * n_part + p];
        row_gs[r] = s;
    }
}

// dL/d weight of this rank's (token, expert) pairs, pulled from the experts' owners: gs_MK[m, k] for token m's k-th
// expert.
__global__ void ep_pull_gs_compact_kernel(PeerPtrs row_gs, const int* __restrict__ home_pos,
                                          const int* __restrict__ home_tile_expert,
                                          const int* __restrict__ remote_row, int Nl, int total,
                                          float* __restrict__ gs_MK) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int pr = home_pos[i];
        const int e = home_tile_expert[pr / TILE_M];
        const float* src = static_cast<const float*>(row_gs.p[e / Nl]) + remote_row[pr];
        float v;
        asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(src));
        gs_MK[i] = v;
    }
}

static int fill_peers(PeerPtrs& out, void* const* ptrs, int world) {
    if (ptrs == nullptr) {
        for (int i = 0; i < EP_MAX_RANKS; ++i) out.p[i] = nullptr;
        return MOMOE_OK;
    }
    for (int i = 0; i < EP_MAX_RANKS; ++i) out.p[i] = i < world ? ptrs[i] : nullptr;
    for (int i = 0; i < world; ++i)
        if (out.p[i] == nullptr) return MOMOE_ERR_ARG;
    return MOMOE_OK;
}

}  // namespace momoe

using namespace momoe;
#define EP_LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? MOMOE_OK : MOMOE_ERR_CUDA)
#define EP_API extern "C" __attribute__((visibility("default")))

EP_API int64_t momoe_ep_set_wait_limit(int64_t sm_cycles) {
    const long long before = g_flag_wait_cycles;
    if (sm_cycles > 0) g_flag_wait_cycles = sm_cycles;
    return before;
}

EP_API int momoe_ep_publish_counts(const int64_t* sizes_N, int32_t N, void* const* peer_counts,
                                   void* const* peer_flags, int32_t world, int32_t rank, uint32_t epoch,
                                   int32_t* status, momoe_stream_t stream) {
    if (sizes_N == nullptr || status == nullptr || N <= 0 || N > 1024) return MOMOE_ERR_ARG;
    if (world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world || N % world != 0) return MOMOE_ERR_ARG;
    PeerPtrs c, f;
    if (peer_counts == nullptr || peer_flags == nullptr) return MOMOE_ERR_ARG;
    if (fill_peers(c, peer_counts, world) != MOMOE_OK || fill_peers(f, peer_flags, world) != MOMOE_OK)
        return MOMOE_ERR_ARG;
    ep_publish_counts_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const long long*>(sizes_N), N, c, f, world, rank, epoch, status, g_flag_wait_cycles);
    return EP_LAUNCH_OK();
}

EP_API int momoe_ep_barrier(void* const* peer_flags, int32_t world, int32_t rank, uint32_t epoch, int32_t* status,
                            momoe_stream_t stream) {
    if (peer_flags == nullptr || status == nullptr) return MOMOE_ERR_ARG;
    if (world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world) return MOMOE_ERR_ARG;
    PeerPtrs f;
    if (fill_peers(f, peer_flags, world) != MOMOE_OK) return MOMOE_ERR_ARG;
    ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, world, rank, epoch, status,
                                                                        g_flag_wait_cycles);
    return EP_LAUNCH_OK();
}

EP_API int momoe_ep_plan(const int32_t* counts_RN, int32_t world, int32_t rank, int32_t N, double save_percent,
                         int64_t cap_rows, int32_t* dst_base_N, int64_t* sizes_global_N, int32_t* local_count,
                         int32_t* pad_off, int32_t* tile_expert, int32_t* pair_info, int32_t* sched, int32_t* status,
                         momoe_stream_t stream) {
    if (counts_RN == nullptr || dst_base_N == nullptr || sizes_global_N == nullptr || local_count == nullptr ||
        pad_off == nullptr || tile_expert == nullptr || pair_info == nullptr || sched == nullptr || status == nullptr)
        return MOMOE_ERR_ARG;
    if (world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world || N <= 0 || N > 1024 || N % world != 0)
        return MOMOE_ERR_ARG;
    if (cap_rows <= 0 || cap_rows % TILE_M != 0 || cap_rows > 0x7fffffffLL || save_percent < 0 || save_percent > 100)
        return MOMOE_ERR_ARG;
    ep_plan_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        counts_RN, world, rank, N, save_percent, cap_rows, static_cast<int>(cap_rows / TILE_M), dst_base_N,
        reinterpret_cast<long long*>(sizes_global_N), local_count, pad_off, tile_expert, pair_info, sched, status, 0,
        nullptr, nullptr);
    return EP_LAUNCH_OK();
}

EP_API int momoe_ep_plan_split(const int32_t* counts_RN, int32_t world, int32_t rank, int32_t N, double save_percent,
                               int64_t cap_rows, int32_t* dst_base_N, int64_t* sizes_global_N, int32_t* local_count,
                               int32_t* pad_off, int32_t* tile_expert, int32_t* pair_info, int32_t* sched,
                               int32_t split_expert, int32_t* pair_info_parts, int32_t* sched_parts, int32_t* status,
                               momoe_stream_t stream) {
    if (counts_RN == nullptr || dst_base_N == nullptr || sizes_global_N == nullptr || local_count == nullptr ||
        pad_off == nullptr || tile_expert == nullptr || pair_info == nullptr || sched == nullptr || status == nullptr ||
        pair_info_parts == nullptr || sched_parts == nullptr)
        return MOMOE_ERR_ARG;
    if (world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world || N <= 0 || N > 1024 || N % world != 0)
        return MOMOE_ERR_ARG;
    if (cap_rows <= 0 || cap_rows % TILE_M != 0 || cap_rows > 0x7fffffffLL || save_percent < 0 || save_percent > 100)
        return MOMOE_ERR_ARG;
    if (split_expert < 0 || split_expert > N / world) return MOMOE_ERR_ARG;
    ep_plan_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        counts_RN, world, rank, N, save_percent, cap_rows, static_cast<int>(cap_rows / TILE_M), dst_base_N,
        reinterpret_cast<long long*>(sizes_global_N), local_count, pad_off, tile_expert, pair_info, sched, status,
        split_expert, pair_info_parts, sched_parts);
    return EP_LAUNCH_OK();
}

static int dispatch_rows_impl(const momoe_plan_t* home, const void* src, int32_t cols, const int32_t* dst_base_N,
                              int32_t experts_per_rank, void* const* peer_rows, void* const* peer_row_weight,
                              int32_t* remote_row, int32_t world, int32_t rank, const int32_t* local_count,
                              const int32_t* local_pad_off, int32_t e_lo, int32_t e_hi, int32_t max_blocks,
                              momoe_stream_t stream) {
    if (home == nullptr || src == nullptr || dst_base_N == nullptr || peer_rows == nullptr || local_count == nullptr ||
        local_pad_off == nullptr || home->row_token == nullptr || home->tile_expert == nullptr ||
        home->pad_off == nullptr || home->sched == nullptr || home->row_weight == nullptr)
        return MOMOE_ERR_ARG;
    if (cols <= 0 || cols % 8 != 0) return MOMOE_ERR_UNSUPPORTED;
    if (world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world || experts_per_rank <= 0) return MOMOE_ERR_ARG;
    if (e_lo < 0 || e_hi > experts_per_rank || e_lo > e_hi) return MOMOE_ERR_ARG;
    PeerPtrs r, w;
    if (fill_peers(r, peer_rows, world) != MOMOE_OK || fill_peers(w, peer_row_weight, world) != MOMOE_OK)
        return MOMOE_ERR_ARG;
    const int grid = max_blocks > 0 ? max_blocks : sm_count() * 8;
    uintptr_t align = reinterpret_cast<uintptr_t>(src);
    for (int i = 0; i < world; ++i) align |= reinterpret_cast<uintptr_t>(r.p[i]);
    const bool wide = (cols % 16 == 0) && (align & 31) == 0;   // 256-bit stores need 32-byte aligned rows
    share_sm_with_gemm<ep_dispatch_rows_kernel>();
    ep_dispatch_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), home->row_token, home->tile_expert, home->pad_off, home->row_weight,
        dst_base_N, experts_per_rank, cols / 8, r, w, remote_row, rank, world, local_count, local_pad_off, wide,
        home->status, e_lo, e_hi);
    return EP_LAUNCH_OK();
}

EP_API int momoe_ep_dispatch_rows(const momoe_plan_t* home, const void* src, int32_t cols, const int32_t* dst_base_N,
                                  int32_t experts_per_rank, void* const* peer_rows, void* const* peer_row_weight,
                                  int32_t* remote_row, int32_t world, int32_t rank, const int32_t* local_count,
                                  const int32_t* local_pad_off, int32_t max_blocks, momoe_stream_t stream) {
    return dispatch_rows_impl(home, src, cols, dst_base_N, experts_per_rank, peer_rows, peer_row_weight, remote_row,
                              world, rank, local_count, local_pad_off, 0, experts_per_rank, max_blocks, stream);
}

EP_API int momoe_ep_dispatch_rows_range(const momoe_plan_t* home, const void* src, int32_t cols,
                                        const int32_t* dst_base_N, int32_t experts_per_rank, void* const* peer_rows,
                                        void* const* peer_row_weight, int32_t* remote_row, int32_t world, int32_t rank,
                                        const int32_t* local_count, const int32_t* local_pad_off, int32_t expert_lo,
                                        int32_t expert_hi, int32_t max_blocks, momoe_stream_t stream) {
    return dispatch_rows_impl(home, src, cols, dst_base_N, experts_per_rank, peer_rows, peer_row_weight, remote_row,
                              world, rank, local_count, local_pad_off, expert_lo, expert_hi, max_blocks, stream);
}

EP_API int momoe_ep_pull_rows(const momoe_plan_t* home, void* const* peer_rows, const int32_t* remote_row,
                              int32_t experts_per_rank, int32_t cols, void* staged_rows, int32_t world, int32_t rank,
                              int32_t expert_lo, int32_t expert_hi, int32_t max_blocks, momoe_stream_t stream) {
    if (home == nullptr || peer_rows == nullptr || remote_row == nullptr || staged_rows == nullptr ||
        home->row_token == nullptr || home->pad_off == nullptr)
        return MOMOE_ERR_ARG;
    if (cols <= 0 || cols % 8 != 0) return MOMOE_ERR_UNSUPPORTED;
    if (world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world || experts_per_rank <= 0) return MOMOE_ERR_ARG;
    if (expert_lo < 0 || expert_hi > experts_per_rank || expert_lo > expert_hi) return MOMOE_ERR_ARG;
    PeerPtrs r;
    if (fill_peers(r, peer_rows, world) != MOMOE_OK) return MOMOE_ERR_ARG;
    const int grid = max_blocks > 0 ? max_blocks : sm_count() * 8;
    share_sm_with_gemm<ep_pull_rows_kernel>();
    ep_pull_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        r, home->row_token, home->pad_off, remote_row, experts_per_rank, cols / 8, static_cast<uint4*>(staged_rows),
        rank, world, expert_lo, expert_hi);
    return EP_LAUNCH_OK();
}

EP_API int momoe_ep_combine_rows_staged(const momoe_plan_t* home, void* const* peer_rows, const int32_t* remote_row,
                                        int32_t experts_per_rank, int32_t cols, void* dst, int32_t world,
                                        const void* staged_rows, int32_t expert_lo, int32_t expert_hi,
                                        int32_t max_blocks, momoe_stream_t stream) {
    if (home == nullptr || peer_rows == nullptr || remote_row == nullptr || dst == nullptr || home->pos_MK == nullptr ||
        home->tile_expert == nullptr || staged_rows == nullptr)
        return MOMOE_ERR_ARG;
    if (cols <= 0 || cols % 8 != 0) return MOMOE_ERR_UNSUPPORTED;
    if (world < 1 || world > EP_MAX_RANKS || experts_per_rank <= 0) return MOMOE_ERR_ARG;
    if (expert_lo < 0 || expert_hi > experts_per_rank || expert_lo > expert_hi) return MOMOE_ERR_ARG;
    PeerPtrs r;
    if (fill_peers(r, peer_rows, world) != MOMOE_OK) return MOMOE_ERR_ARG;
    const int vec = cols / 8;
    const long long total = static_cast<long long>(home->M) * vec;
    int blocks = static_cast<int>((total + 255) / 256);
    const int cap = max_blocks > 0 ? max_blocks : sm_count() * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint4* d = static_cast<uint4*>(dst);
    const uint4* sg = static_cast<const uint4*>(staged_rows);
#define MOMOE_COMBINE_STAGED(KT)                                                                                      \
    share_sm_with_gemm<ep_combine_rows_staged_kernel<KT>>();                                                         \
    ep_combine_rows_staged_kernel<KT><<<blocks, 256, 0, st>>>(r, home->pos_MK, home->tile_expert, remote_row,         \
                                                              experts_per_rank, home->M, home->K, vec, d, sg,         \
                                                              expert_lo, expert_hi)
    switch (home->K) {
        case 2: MOMOE_COMBINE_STAGED(2); break;
        case 4: MOMOE_COMBINE_STAGED(4); break;
        case 6: MOMOE_COMBINE_STAGED(6); break;
        case 8: MOMOE_COMBINE_STAGED(8); break;
        default: MOMOE_COMBINE_STAGED(0); break;
    }
#undef MOMOE_COMBINE_STAGED
    return EP_LAUNCH_OK();
}

EP_API int momoe_ep_combine_rows(const momoe_plan_t* home, void* const* peer_rows, const int32_t* remote_row,
                                 int32_t experts_per_rank, int32_t cols, void* dst, int32_t world, int32_t max_blocks,
                                 momoe_stream_t stream) {
    if (home == nullptr || peer_rows == nullptr || remote_row == nullptr || dst == nullptr || home->pos_MK == nullptr ||
        home->tile_expert == nullptr)
        return MOMOE_ERR_ARG;
    if (cols <= 0 || cols % 8 != 0) return MOMOE_ERR_UNSUPPORTED;
    if (world < 1 || world > EP_MAX_RANKS || experts_per_rank <= 0) return MOMOE_ERR_ARG;
    PeerPtrs r;
    if (fill_peers(r, peer_rows, world) != MOMOE_OK) return MOMOE_ERR_ARG;
    const int vec = cols / 8;
    const long long total = static_cast<long long>(home->M) * vec;
    int blocks = static_cast<int>((total + 255) / 256);
    const int cap = max_blocks > 0 ? max_blocks : sm_count() * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint4* d = static_cast<uint4*>(dst);
    switch (home->K) {
        case 2: share_sm_with_gemm<ep_combine_rows_kernel<2>>(); ep_combine_rows_kernel<2><<<blocks, 256, 0, st>>>(r, home->pos_MK, home->tile_expert, remote_row, experts_per_rank, home->M, vec, d); break;
        case 4: share_sm_with_gemm<ep_combine_rows_kernel<4>>(); ep_combine_rows_kernel<4><<<blocks, 256, 0, st>>>(r, home->pos_MK, home->tile_expert, remote_row, experts_per_rank, home->M, vec, d); break;
        case 6: share_sm_with_gemm<ep_combine_rows_kernel<6>>(); ep_combine_rows_kernel<6><<<blocks, 256, 0, st>>>(r, home->pos_MK, home->tile_expert, remote_row, experts_per_rank, home->M, vec, d); break;
        case 8: share_sm_with_gemm<ep_combine_rows_kernel<8>>(); ep_combine_rows_kernel<8><<<blocks, 256, 0, st>>>(r, home->pos_MK, home->tile_expert, remote_row, experts_per_rank, home->M, vec, d); break;
        default: share_sm_with_gemm<ep_combine_rows_generic_kernel>(); ep_combine_rows_generic_kernel<<<blocks, 256, 0, st>>>(r, home->pos_MK, home->tile_expert, remote_row, experts_per_rank, home->M, home->K, vec, d); break;
    }
    return EP_LAUNCH_OK();
}

EP_API int momoe_ep_reduce_gs(const float* gs_part, int32_t n_part, const int32_t* sched, float* row_gs,
                              momoe_stream_t stream) {
    if (gs_part == nullptr || sched == nullptr || row_gs == nullptr || n_part <= 0) return MOMOE_ERR_ARG;
    ep_reduce_gs_kernel<<<sm_count() * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(gs_part, n_part, sched, row_gs);
    return EP_LAUNCH_OK();
}

EP_API int momoe_ep_pull_gs_compact(const momoe_plan_t* home, void* const* peer_row_gs, const int32_t* remote_row,
                                    int32_t experts_per_rank, float* gs_MK, int32_t world, momoe_stream_t stream) {
    if (home == nullptr || peer_row_gs == nullptr || remote_row == nullptr || gs_MK == nullptr ||
        home->pos_MK == nullptr || home->tile_expert == nullptr)
        return MOMOE_ERR_ARG;
    if (world < 1 || world > EP_MAX_RANKS || experts_per_rank <= 0) return MOMOE_ERR_ARG;
    PeerPtrs g;
    if (fill_peers(g, peer_row_gs, world) != MOMOE_OK) return MOMOE_ERR_ARG;
    ep_pull_gs_compact_kernel<<<sm_count() * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        g, home->pos_MK, home->tile_expert, remote_row, experts_per_rank, home->M * home->K, gs_MK);
    return EP_LAUNCH_OK();
}
