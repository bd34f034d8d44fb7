/* C ABI of libmomoe_b200.so: the B200 (sm_100a) implementation of the MoMoE layer hot path.
 *
 * Each entry point replaces one piece of the reference's Python/Triton path; the reference location it
 * stands in for is cited as file:line relative to the reference project root.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless stated otherwise; bf16 tensors are passed as `const void*`;
 *  - no entry point allocates device memory or synchronises the host with the device; all work is queued on
 *    the `stream` argument (a cudaStream_t passed as void*);
 *  - return value: 0 on success, negative when the arguments are rejected on the host (nothing is launched);
 *  - problems that only the device can detect (a wait that ran out, a token without exactly K experts) are
 *    written as a positive code into the caller's int32 `status` word, which must be zeroed by the caller;
 *  - "expert-major" buffers hold one row per (token, expert) pair, grouped by expert in ascending expert id and,
 *    inside an expert, ascending token id.  Every expert segment starts at a multiple of 128 rows (padding rows
 *    are zero), so every 128-row tile belongs to exactly one expert.  `momoe_sorted_rows_capacity` gives the
 *    number of rows such a buffer must have.
 */
#ifndef MOMOE_B200_H
#define MOMOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* momoe_stream_t;

/* Routing plan of one forward pass: dimensions plus the device tables written by momoe_build_permutation. */
typedef struct momoe_plan {
    int32_t M;                   /* tokens (B*S) */
    int32_t N;                   /* experts */
    int32_t K;                   /* experts per token, shared experts included */
    int32_t D;                   /* embedding dim */
    int32_t H;                   /* intermediate dim */
    int32_t reserved;
    int64_t rows_capacity;       /* rows of every expert-major buffer (momoe_sorted_rows_capacity) */
    const int32_t* sched;        /* int32[8]: [0] 128-row tiles in use, [1] tiles whose a,b are saved, [2] padded rows,
                                    [3] tile pairs */
    const int32_t* tile_expert;  /* int32[momoe_tile_capacity]: expert of each tile */
    const int32_t* pad_off;      /* int32[N+1]: first padded row of each expert */
    const int32_t* row_token;    /* int32[rows_capacity]: token of each padded row, -1 on padding rows */
    const float* row_weight;     /* float[rows_capacity]: routing weight of each padded row, 0 on padding rows */
    const int32_t* pos_MK;       /* int32[M*K]: padded row of token m's k-th expert (ascending expert id) */
    int32_t* status;             /* device int32 error word, zeroed by the caller */
    const int32_t* pair_info;    /* int32[momoe_tile_capacity]: for each pair of consecutive tiles of one expert,
                                    first tile * 2 + (1 if the pair has a second tile); the grouped GEMMs give one
                                    pair to two cooperating thread blocks */
} momoe_plan_t;

int momoe_version(void);

/* Rows / tiles an expert-major buffer needs for M tokens, K experts each, N experts (host arithmetic only). */
int64_t momoe_sorted_rows_capacity(int32_t M, int32_t K, int32_t N);
int64_t momoe_tile_capacity(int32_t M, int32_t K, int32_t N);

/* Router after the gate GEMM: fp32 softmax over the N-Ks gating experts and over the Ks shared experts,
 * top-(K-Ks) of probability + bias (ties: lowest expert id), renormalisation.
 * Replaces momoe/topk_router.py:96-120.
 *   logits_MN   bf16 [M,N] contiguous;  biases_N fp32 [N] (entries of shared experts are not read)
 *   topk_idx_MK int32 [M,K] ascending expert ids (shared experts last);  topk_w_MK fp32 [M,K] their weights
 *   optional dense outputs (all NULL or all non-NULL): mask_NM int32 [N,M], s_MN fp32 [M,N] (the reference's
 *   s_NM is its transpose view), s_postsoft_MN fp32 [M,N];
 *   optional normalisers (both NULL or both non-NULL; required with the dense outputs): Ng_M fp32 [M] = sum of the
 *   selected gating probabilities, Ks_M fp32 [M] = sum of the shared experts' probabilities. */
int momoe_route_topk(const void* logits_MN, const float* biases_N, int32_t M, int32_t N, int32_t K, int32_t Ks,
                     int32_t* topk_idx_MK, float* topk_w_MK, int32_t* mask_NM, float* s_MN, float* s_postsoft_MN,
                     float* Ng_M, float* Ks_M, momoe_stream_t stream);

/* Compact form of an external router's dense mask_NM / s_NM (any strides, in elements).
 * Replaces the mask scan of momoe/momoe.py:760-815.  A token without exactly K experts sets *status. */
int momoe_topk_from_mask(const int32_t* mask_NM, int64_t mask_stride_n, int64_t mask_stride_m, const float* s_NM,
                         int64_t s_stride_n, int64_t s_stride_m, int32_t M, int32_t N, int32_t K,
                         int32_t* topk_idx_MK, float* topk_w_MK, int32_t* status, momoe_stream_t stream);

/* Kernels momoe_build_permutation launches for this problem: 1 (up to 1024 tokens and 256 experts: the three passes
 * and the initialisation of the padding rows run in one thread block) or 3 (+ two memsets).  Host arithmetic only. */
int momoe_permutation_launches(int32_t M, int32_t N, int32_t K);

/* Expert-major permutation from the compact routing.  Replaces momoe/momoe.py:821-842 (find_used_experts).
 * Outputs identical to the reference: sizes_N int64 [N], cumsums_N1 int32 [N+1], idx_Msum int32 [M*K],
 * which_Msum int32 [M*K] (slot = rank of the expert among the token's experts).  Plus the padded tables of
 * momoe_plan_t.  save_rows = int(M*K*save_percent/100) (momoe/momoe.py:251); sched[1] receives the number of
 * leading tiles that lie entirely below it (the tile rule of momoe/momoe.py:486). */
size_t momoe_permutation_workspace_bytes(int32_t M, int32_t N, int32_t K);
int momoe_build_permutation(const int32_t* topk_idx_MK, const float* topk_w_MK, int32_t M, int32_t N, int32_t K,
                            int64_t save_rows, int64_t* sizes_N, int32_t* cumsums_N1, int32_t* idx_Msum,
                            int32_t* which_Msum, int32_t* pad_off, int32_t* tile_expert, int32_t* pair_info,
                            int32_t* sched, int32_t* row_token, float* row_weight, int32_t* pos_MK,
                            int64_t rows_capacity, void* workspace, size_t workspace_bytes, int32_t* status,
                            momoe_stream_t stream);

/* The same permutation builder for callers that cannot provide a workspace.  It has no counterpart in the
 * reference.  Some hosts of this library are not able to allocate device memory when they route tokens: an
 * inference server whose own pool took all of HBM at start-up, a latency-critical loop that must avoid the device
 * synchronisation an allocation implies, a plug-in that only ever receives its input and output tensors.  Here
 * the chunk histogram lives in a 1 MiB array inside the library image (every GPU that loads the library holds
 * that 1 MiB until the process exits), and the call allocates nothing.
 *   Limit: ceil(M/64) * N <= 262144 (for example 65536 tokens x 256 experts); larger problems return -4 and
 *   launch nothing.  All other arguments, outputs and return codes are those of momoe_build_permutation.
 *   The first call on each device looks up the array's device address (a runtime call that may load the module):
 *   make that first call outside any stream capture.
 *   All calls on a device share the one array and it keeps the last call's contents; the kernels overwrite every
 *   entry they later read, so nothing needs clearing, but two calls that overlap on the GPU (different streams
 *   without ordering between them) race on it and corrupt each other's result. */
int momoe_build_permutation_static(const int32_t* topk_idx_MK, const float* topk_w_MK, int32_t M, int32_t N,
                                   int32_t K, int64_t save_rows, int64_t* sizes_N, int32_t* cumsums_N1,
                                   int32_t* idx_Msum, int32_t* which_Msum, int32_t* pad_off, int32_t* tile_expert,
                                   int32_t* pair_info, int32_t* sched, int32_t* row_token, float* row_weight,
                                   int32_t* pos_MK, int64_t rows_capacity, int32_t* status, momoe_stream_t stream);

/* dst[r,:] = src[row_token[r],:] (zeros on padding rows), bf16, `cols` columns (multiple of 8).  Each source row is
 * read once and stored to the token's K rows (plan->pos_MK); with plan->pos_MK == NULL the rows are fetched one by
 * one from plan->row_token alone.
 * Replaces the row gathers of momoe/momoe.py:116-118 and :298-350. */
int momoe_gather_rows(const momoe_plan_t* plan, const void* src, int32_t cols, void* dst_sorted,
                      momoe_stream_t stream);

/* dst[m,:] = bf16( sum_k float(src_sorted[pos_MK[m,k],:]) ).  Replaces the K-slab scatter + `sum(dim=0)` of
 * momoe/momoe.py:234-237,290 and :679-681,754. */
int momoe_combine_rows(const momoe_plan_t* plan, const void* src_sorted, int32_t cols, void* dst,
                       momoe_stream_t stream);

/* Up/gate grouped GEMM + SwiGLU: a = x W1[e][:, :H], b = x W1[e][:, H:], h = bf16(a * b * sigmoid(b)).
 * Replaces momoe/momoe.py:69-152.
 *   ab_mode 0: only h is written.
 *   ab_mode 1: h, and bf16 a,b of the saved tiles (tile < sched[1]) at row tile*128 of a_out/b_out.
 *   ab_mode 2: recomputation for the backward pass: only tiles >= sched[1] are processed, a,b go to row
 *              (tile - sched[1])*128 of a_out/b_out; h_sorted may be NULL. */
int momoe_up_swiglu(const momoe_plan_t* plan, const void* x_sorted, const void* W1_ND2H, void* h_sorted,
                    void* a_out, void* b_out, int32_t ab_mode, momoe_stream_t stream);

/* momoe_up_swiglu with the row gather folded into the GEMM's operand loads, as the reference's kernel does
 * (momoe/momoe.py:116-118: `x` rows are fetched through the expert-major index inside lin1_kernel).  x_MD is the
 * token-major input bf16 [plan->M, D]; row r of the A operand is x_MD[plan->row_token[r], :], fetched four rows per
 * TMA row-gather load.  No expert-major copy of x exists.  A padding row (row_token -1) repeats the first row of its
 * 128-row tile, so its h, a, b are those of a real row of the same expert, not zeros; everything downstream
 * multiplies padding rows by their zero routing weight.  Other arguments as momoe_up_swiglu. */
int momoe_up_swiglu_tokens(const momoe_plan_t* plan, const void* x_MD, const void* W1_ND2H, void* h_sorted,
                           void* a_out, void* b_out, int32_t ab_mode, momoe_stream_t stream);

/* Down grouped GEMM with the routing weight in the epilogue: y_sorted[r,:] = bf16(w[r] * (h[r,:] W2[e])).
 * Replaces momoe/momoe.py:161-237. */
int momoe_down_scale(const momoe_plan_t* plan, const void* h_sorted, const void* W2_NHD, void* y_sorted,
                     momoe_stream_t stream);

/* The two forward GEMMs for small token batches (inference: a few rows per expert, nothing kept for a backward
 * pass).  Same inputs, outputs and arithmetic as momoe_up_swiglu with ab_mode 0 and momoe_down_scale; the weights
 * are the 128-row side of the MMA and 32 tokens its N side, so that shared memory holds weights in flight instead of
 * padding rows and the kernels run at the speed the weights cross HBM.  Only the 32-row blocks of a tile that hold
 * real rows are written (blocks of padding rows keep whatever the buffer held).  Replace momoe/momoe.py:69-152 and
 * :161-237 for forward-only calls. */
int momoe_up_swiglu_decode(const momoe_plan_t* plan, const void* x_sorted, const void* W1_ND2H, void* h_sorted,
                           momoe_stream_t stream);
int momoe_down_scale_decode(const momoe_plan_t* plan, const void* h_sorted, const void* W2_NHD, void* y_sorted,
                            momoe_stream_t stream);

/* Backward of the down projection fused with the SwiGLU backward.  Replaces momoe/momoe.py:421-535 and the
 * G_s reduction of :684-703.  With Gh = g_sorted W2[e]^T (g_sorted is the UN-weighted gathered upstream
 * gradient) and a,b taken from the saved buffers (tile < sched[1]) or the recomputed ones:
 *   gz_sorted [rows,2H] = bf16[ w*Gh*b*sig(b) | w*Gh*a*sig(b)*(1+b*(1-sig(b))) ]
 *   hs_sorted [rows,H]  = bf16( w * bf16(a*b*sig(b)) )           (left operand of the W2 gradient)
 *   gs_part   [rows,2*ceil(H/256)] fp32 partial sums of <Gh, bf16(a*b*sig(b))> (their sum is dL/ds). */
int momoe_dgrad2_swiglu_bwd(const momoe_plan_t* plan, const void* g_sorted, const void* W2_NHD,
                            const void* a_saved, const void* b_saved, const void* a_recomp, const void* b_recomp,
                            void* gz_sorted, void* hs_sorted, float* gs_part, momoe_stream_t stream);

/* momoe_dgrad2_swiglu_bwd reading the upstream gradient token-major: g_MD bf16 [plan->M, D], rows fetched through
 * plan->row_token inside the GEMM.  Replaces the pre-gather of momoe/momoe.py:298-350 (making_nice_scatter_kernel)
 * together with :421-535.  gs_part of padding rows is unspecified (nothing reads it). */
int momoe_dgrad2_swiglu_bwd_tokens(const momoe_plan_t* plan, const void* g_MD, const void* W2_NHD,
                                   const void* a_saved, const void* b_saved, const void* a_recomp,
                                   const void* b_recomp, void* gz_sorted, void* hs_sorted, float* gs_part,
                                   momoe_stream_t stream);

/* gx_sorted = bf16(gz_sorted W1[e]^T).  Replaces the GEMM of momoe/momoe.py:612-681. */
int momoe_dgrad1(const momoe_plan_t* plan, const void* gz_sorted, const void* W1_ND2H, void* gx_sorted,
                 momoe_stream_t stream);

/* dW[e] = bf16( A_e^T B_e ) over the rows of expert e (fp32 accumulation; zero for experts without tokens).
 * A: [rows, X], B: [rows, Y] expert-major bf16.  Replaces momoe/momoe.py:356-412. */
int momoe_wgrad(const momoe_plan_t* plan, const void* a_sorted, int32_t X, const void* b_sorted, int32_t Y,
                void* dW_NXY, momoe_stream_t stream);

/* momoe_wgrad with either operand token-major: when a_is_token_major (b_is_token_major) is non-zero, `a` (`b`) is a
 * bf16 [plan->M, X] ([plan->M, Y]) matrix whose rows are fetched through plan->row_token; the other operand must be
 * expert-major with zero padding rows (hs_sorted and gz_sorted are).  Replaces momoe/momoe.py:356-412 fed by the
 * gathers of :298-350. */
int momoe_wgrad_tokens(const momoe_plan_t* plan, const void* a, int32_t X, int32_t a_is_token_major, const void* b,
                       int32_t Y, int32_t b_is_token_major, void* dW_NXY, momoe_stream_t stream);

/* Dense G_s_NM fp32 [N,M] contiguous (zero where unselected) from the per-row partial sums.
 * Replaces the zero-init + atomics of momoe/momoe.py:721,699-703. */
int momoe_scatter_gs(const momoe_plan_t* plan, const float* gs_part, int32_t n_part, float* G_s_NM,
                     momoe_stream_t stream);

/* Router backward before the two gate GEMMs: renormalisation backward then softmax backward, separately for
 * the gating and the shared group, rounded to bf16.  Replaces momoe/topk_router.py:11-56.
 *   G_s: dL/ds addressed as G_s[n*gs_stride_n + m*gs_stride_m]; output G_logits_MN bf16 [M,N]. */
int momoe_router_backward(const float* G_s, int64_t gs_stride_n, int64_t gs_stride_m, const float* s_postsoft_MN,
                          const float* s_MN, const float* Ng_M, const float* Ks_M, const int32_t* mask_NM,
                          int32_t M, int32_t N, int32_t Ks, void* G_logits_MN, momoe_stream_t stream);

/* The same router backward without any dense [N,M] tensor: reads the per-row partial sums that
 * momoe_dgrad2_swiglu_bwd wrote (summed in the order momoe_scatter_gs uses), the compact routing of
 * momoe_route_topk and its two normalisers; unselected experts get a zero gradient.  Output G_logits_MN bf16 [M,N].
 * plan->pos_MK may be NULL: gs_part is then already in the routing's compact order, row m*K+k for token m's k-th
 * expert (with n_part = 1 this is dL/d topk_w).
 * Replaces momoe/momoe.py:721,699-703 (dense G_s) together with momoe/topk_router.py:11-56.  K <= 32. */
int momoe_router_backward_compact(const momoe_plan_t* plan, const float* gs_part, int32_t n_part,
                                  const int32_t* topk_idx_MK, const float* topk_w_MK, const float* Ng_M,
                                  const float* Ks_M, int32_t Ks, void* G_logits_MN, momoe_stream_t stream);

/* Aux-loss-free load balancing in place: biases_N[e] += rate * sign(c_avg - sizes_N[e]) for e < N-Ks, in fp32 (the
 * shared experts' entries, -inf, are not touched).  Replaces the three torch ops of momoe/sample_moe.py:64-66. */
int momoe_bias_update(float* biases_N, const int64_t* sizes_N, int32_t N, int32_t Ks, float c_avg, float rate,
                      momoe_stream_t stream);

/* ------------------------------------------------------------------------------------------------------------
 * Expert parallelism over peer memory (no counterpart in the reference, whose README lists expert parallelism as
 * unsupported).  R <= 8 ranks of one NVLink node, one process per GPU; rank r owns experts [r*N/R, (r+1)*N/R).
 * `peer_*` arguments are HOST arrays of R device pointers: entry p is rank p's buffer, mapped into this process
 * (entry [rank] is the local one).  The flag arrays (uint32[8] per rank) must start zeroed; `epoch` must grow by one
 * with every hand-shake, identically on every rank.  Waits on a peer are bounded (status 301 when they run out).
 * ------------------------------------------------------------------------------------------------------------ */

/* Limit of every wait on a peer's flag, in SM clock cycles (default 4e9, about two seconds); values <= 0 leave it
 * unchanged.  Returns the previous limit.  A process-wide host-side setting, read when a hand-shake is launched.  A
 * wait that runs out writes status 301 and the kernel returns normally; once 301 is recorded momoe_ep_dispatch_rows
 * sends nothing. */
int64_t momoe_ep_set_wait_limit(int64_t sm_cycles);

/* Store this rank's per-expert token counts (sizes_N of momoe_build_permutation) into row `rank` of every peer's
 * int32[R*N] counts matrix, then hand-shake: on return (in stream order) this rank's matrix is complete. */
int momoe_ep_publish_counts(const int64_t* sizes_N, int32_t N, void* const* peer_counts, void* const* peer_flags,
                            int32_t world, int32_t rank, uint32_t epoch, int32_t* status, momoe_stream_t stream);

/* Hand-shake only: every rank has executed everything it queued before this call. */
int momoe_ep_barrier(void* const* peer_flags, int32_t world, int32_t rank, uint32_t epoch, int32_t* status,
                     momoe_stream_t stream);

/* From the complete counts matrix, on the device: the padded expert-major layout of this rank's expert block
 * (local_count int32[N/R], pad_off int32[N/R+1], tile_expert, pair_info, sched: the tables of momoe_plan_t, with
 * sched[1] following save_percent of the rows this rank received), dst_base_N int32[N] (row inside the owner's layout
 * where this rank's tokens for each expert start; -1 everywhere and status 302 if some rank would exceed cap_rows),
 * and sizes_global_N int64[N] (tokens per expert summed over ranks: the layer's tokens_per_expert_N). */
int momoe_ep_plan(const int32_t* counts_RN, int32_t world, int32_t rank, int32_t N, double save_percent,
                  int64_t cap_rows, int32_t* dst_base_N, int64_t* sizes_global_N, int32_t* local_count,
                  int32_t* pad_off, int32_t* tile_expert, int32_t* pair_info, int32_t* sched, int32_t* status,
                  momoe_stream_t stream);

/* momoe_ep_plan that also cuts this rank's expert block in two parts, local experts [0, split_expert) and
 * [split_expert, N/R), so that the transfers of one part can run while the grouped GEMMs work on the other:
 * pair_info_parts int32[2 * (cap_rows/128)] receives the pair table of part 0 at [0] and of part 1 at
 * [cap_rows/128], sched_parts int32[2*8] the matching schedule words (sched_parts[8*p + 3] = pairs of part p; tile
 * numbers, and with them the boundary of the saved tiles, are those of the whole block).  A momoe_plan_t that points
 * at one part's tables makes the row-tile GEMMs (up, down, dgrad-2, dgrad-1) work on that part's experts only. */
int momoe_ep_plan_split(const int32_t* counts_RN, int32_t world, int32_t rank, int32_t N, double save_percent,
                        int64_t cap_rows, int32_t* dst_base_N, int64_t* sizes_global_N, int32_t* local_count,
                        int32_t* pad_off, int32_t* tile_expert, int32_t* pair_info, int32_t* sched,
                        int32_t split_expert, int32_t* pair_info_parts, int32_t* sched_parts, int32_t* status,
                        momoe_stream_t stream);

/* Gather + send: row src[token,:] of every (token, expert) pair of `home` (this rank's own permutation over all N
 * experts) is stored into the owner's expert-major buffer at dst_base_N[e] + (index among this rank's tokens of e);
 * peer_row_weight (may be NULL) receives the routing weight, remote_row (may be NULL, int32[home rows_capacity])
 * the row used.  Also zeroes the padding rows of this rank's own buffer.
 * max_blocks (here and in momoe_ep_combine_rows): 0 = size the grid for the whole GPU; one block of 256 threads per
 * SM (max_blocks = SM count) is enough to fill NVLink and leaves room for a grouped GEMM, queued on another stream,
 * to run on the same SMs at the same time. */
int momoe_ep_dispatch_rows(const momoe_plan_t* home, const void* src, int32_t cols, const int32_t* dst_base_N,
                           int32_t experts_per_rank, void* const* peer_rows, void* const* peer_row_weight,
                           int32_t* remote_row, int32_t world, int32_t rank, const int32_t* local_count,
                           const int32_t* local_pad_off, int32_t max_blocks, momoe_stream_t stream);

/* momoe_ep_dispatch_rows for the (token, expert) pairs whose expert is one of its owner's local experts
 * [expert_lo, expert_hi) only (and the padding rows of this rank's own experts in that range). */
int momoe_ep_dispatch_rows_range(const momoe_plan_t* home, const void* src, int32_t cols, const int32_t* dst_base_N,
                                 int32_t experts_per_rank, void* const* peer_rows, void* const* peer_row_weight,
                                 int32_t* remote_row, int32_t world, int32_t rank, const int32_t* local_count,
                                 const int32_t* local_pad_off, int32_t expert_lo, int32_t expert_hi,
                                 int32_t max_blocks, momoe_stream_t stream);

/* Receive without reducing: the result rows of this rank's (token, expert) pairs whose expert is one of its owner's
 * local experts [expert_lo, expert_hi) are copied from the owners into staged_rows (bf16 [home rows_capacity, cols],
 * local memory, row index = the pair's row in `home`).  Queued beside the GEMMs of the other experts. */
int momoe_ep_pull_rows(const momoe_plan_t* home, void* const* peer_rows, const int32_t* remote_row,
                       int32_t experts_per_rank, int32_t cols, void* staged_rows, int32_t world, int32_t rank,
                       int32_t expert_lo, int32_t expert_hi, int32_t max_blocks, momoe_stream_t stream);

/* Receive + reduce: dst[m,:] = bf16(sum_k rows@owner(m,k)[remote_row,:]), fp32 accumulation in ascending k. */
int momoe_ep_combine_rows(const momoe_plan_t* home, void* const* peer_rows, const int32_t* remote_row,
                          int32_t experts_per_rank, int32_t cols, void* dst, int32_t world, int32_t max_blocks,
                          momoe_stream_t stream);

/* momoe_ep_combine_rows where the rows of the owners' local experts [expert_lo, expert_hi) were fetched before by
 * momoe_ep_pull_rows and are read from staged_rows; the other rows come from their owners.  Same summation order,
 * so the result is identical bit for bit to momoe_ep_combine_rows. */
int momoe_ep_combine_rows_staged(const momoe_plan_t* home, void* const* peer_rows, const int32_t* remote_row,
                                 int32_t experts_per_rank, int32_t cols, void* dst, int32_t world,
                                 const void* staged_rows, int32_t expert_lo, int32_t expert_hi, int32_t max_blocks,
                                 momoe_stream_t stream);

/* row_gs[r] = sum of the dgrad-2 partial sums of local row r. */
int momoe_ep_reduce_gs(const float* gs_part, int32_t n_part, const int32_t* sched, float* row_gs,
                       momoe_stream_t stream);

/* dL/d routing weight of this rank's (token, expert) pairs, pulled from the owners' row_gs:
 * gs_MK fp32 [M,K], entry (m,k) for token m's k-th expert. */
int momoe_ep_pull_gs_compact(const momoe_plan_t* home, void* const* peer_row_gs, const int32_t* remote_row,
                             int32_t experts_per_rank, float* gs_MK, int32_t world, momoe_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MOMOE_B200_H */
