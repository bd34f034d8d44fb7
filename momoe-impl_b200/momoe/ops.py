"""Host-side plumbing above the C ABI: device buffers (torch), the routing plan, and the forward / backward
sequences of kernel launches.  No arithmetic on tensor contents happens here."""
import ctypes as C
import os

import torch

from . import _lib
from ._lib import lib, ptr, stream_ptr, check

TILE_M = 128
_status_words = {}

# Launch accounting.  LAUNCHES counts kernels queued through the C ABI; when KERNEL_EVENTS is a list, every call
# is bracketed by CUDA events on the launching stream (used by the benchmark for per-kernel device times).
LAUNCHES = 0
KERNEL_EVENTS = None
NVTX = os.environ.get("MOMOE_B200_NVTX", "0") == "1"   # one NVTX range per C-ABI call, for timeline tools


def _call(name, n_kernels, fn, *args):
    global LAUNCHES
    ev = KERNEL_EVENTS
    if ev is not None:
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = fn(*args)
        e1.record()
        ev.append((name, e0, e1))
    elif NVTX:
        torch.cuda.nvtx.range_push(name)
        rc = fn(*args)
        torch.cuda.nvtx.range_pop()
    else:
        rc = fn(*args)
    check(rc, name)
    LAUNCHES += n_kernels


def status_word(device):
    """Per-device int32 word the kernels report device-side problems into (0 = fine)."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _status_words[key]


_STATUS_TEXT = {101: "TMA producer wait timed out", 102: "MMA issuer wait timed out",
                103: "epilogue wait timed out", 201: "a token does not have exactly K experts in mask_NM",
                202: "expert id out of range", 301: "a peer rank did not reach a hand-shake in time",
                302: "expert-parallel buffers too small for this routing (raise capacity_factor)"}


def check_status(device=None):
    """Synchronises and raises if any kernel recorded a device-side problem.  Clears the word."""
    w = status_word(device if device is not None else torch.cuda.current_device())
    v = int(w.item())
    if v != 0:
        w.zero_()
        rep = _status_reports.get(w.device.index)
        if rep is not None:      # a copy of the same code may be on its way to the host: it has been reported now
            torch.cuda.synchronize(w.device)
            rep["posted"] = False
            rep["host"][0] = 0
        raise RuntimeError("momoe device status %d: %s" % (v, _STATUS_TEXT.get(v, "unknown")))


# Asynchronous report of the status word: at the end of a pass the word is copied to pinned host memory with a
# non-blocking copy; the next pass looks at the copy once the copy's event has completed and raises if a kernel left a
# code there.  The host is never synchronised, so an error surfaces one pass late (MOMOE_B200_CHECK=1 reports it at
# the end of the same pass, with a synchronisation).  MOMOE_B200_ASYNC_STATUS=0 switches the report off (the word can
# still be read with check_status); it is also skipped while a CUDA graph is being captured.
ASYNC_STATUS = os.environ.get("MOMOE_B200_ASYNC_STATUS", "1") == "1"
_status_reports = {}


def status_post(device):
    """Queue a copy of the device's status word to pinned host memory (no host synchronisation)."""
    if not ASYNC_STATUS or torch.cuda.is_current_stream_capturing():
        return
    w = status_word(device)
    key = w.device.index
    rep = _status_reports.get(key)
    if rep is None:
        rep = _status_reports[key] = dict(host=torch.zeros(1, dtype=torch.int32).pin_memory(),
                                          event=torch.cuda.Event(), posted=False)
    elif rep["posted"] and not rep["event"].query():
        return          # the previous report is still on its way; it will carry any code that is set by then or later
    rep["host"].copy_(w, non_blocking=True)
    rep["event"].record(torch.cuda.current_stream(w.device))
    rep["posted"] = True


def status_poll(device):
    """Raise if a report posted by an earlier pass has arrived with a device-side error code.  Never blocks."""
    d = torch.device(device)
    if not ASYNC_STATUS or d.type != "cuda" or not _status_reports:
        return
    if torch.cuda.is_current_stream_capturing():
        return
    key = d.index if d.index is not None else torch.cuda.current_device()
    rep = _status_reports.get(key)
    if rep is None or not rep["posted"] or not rep["event"].query():
        return
    rep["posted"] = False
    v = int(rep["host"][0])
    if v != 0:
        rep["host"][0] = 0
        status_word(device).zero_()
        raise RuntimeError("momoe device status %d (reported by an earlier pass): %s" % (v, _STATUS_TEXT.get(v, "unknown")))


def save_rows(Msum, save_percent):
    return int(Msum * save_percent / 100.0)


class RoutingPlan:
    """Device tables of one routing decision (see momoe_plan_t) plus the reference-visible permutation."""

    def __init__(self, M, N, K, D, H, device, save_percent=0.0):
        self.M, self.N, self.K, self.D, self.H = M, N, K, D, H
        self.device = device
        self.Msum = M * K
        self.save_rows = save_rows(self.Msum, save_percent)
        self.rows_capacity = int(lib.momoe_sorted_rows_capacity(M, K, N))
        self.tile_capacity = int(lib.momoe_tile_capacity(M, K, N))
        self.saved_tile_capacity = min(self.tile_capacity, self.save_rows // TILE_M + N) if self.save_rows > 0 else 0
        self.recomp_tile_capacity = min(self.tile_capacity, (self.Msum - self.save_rows) // TILE_M + N + 1)
        i32 = dict(dtype=torch.int32, device=device)
        self.sizes = torch.empty(N, dtype=torch.int64, device=device)
        self.cumsums = torch.empty(N + 1, **i32)
        self.idx = torch.empty(self.Msum, **i32)
        self.which = torch.empty(self.Msum, **i32)
        self.pad_off = torch.empty(N + 1, **i32)
        self.tile_expert = torch.empty(self.tile_capacity, **i32)
        self.pair_info = torch.empty(self.tile_capacity, **i32)
        self.sched = torch.empty(8, **i32)
        self.row_token = torch.empty(self.rows_capacity, **i32)
        self.row_weight = torch.empty(self.rows_capacity, dtype=torch.float32, device=device)
        self.pos = torch.empty(self.Msum, **i32)
        self.status = status_word(device)
        self.topk_idx = None
        self.topk_w = None
        self.c = _lib.Plan(M=M, N=N, K=K, D=D, H=H, reserved=0, rows_capacity=self.rows_capacity,
                           sched=self.sched.data_ptr(), tile_expert=self.tile_expert.data_ptr(),
                           pad_off=self.pad_off.data_ptr(), row_token=self.row_token.data_ptr(),
                           row_weight=self.row_weight.data_ptr(), pos_MK=self.pos.data_ptr(),
                           status=self.status.data_ptr(), pair_info=self.pair_info.data_ptr())

    @property
    def ref(self):
        return C.byref(self.c)

    def build(self, topk_idx, topk_w):
        self.topk_idx, self.topk_w = topk_idx, topk_w
        nbytes = int(lib.momoe_permutation_workspace_bytes(self.M, self.N, self.K))
        ws = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=self.device)
        _call("momoe_build_permutation", int(lib.momoe_permutation_launches(self.M, self.N, self.K)),
              lib.momoe_build_permutation, ptr(topk_idx), ptr(topk_w), self.M, self.N, self.K, self.save_rows,
                                          ptr(self.sizes), ptr(self.cumsums), ptr(self.idx), ptr(self.which),
                                          ptr(self.pad_off), ptr(self.tile_expert), ptr(self.pair_info), ptr(self.sched),
                                          ptr(self.row_token), ptr(self.row_weight), ptr(self.pos),
                                          self.rows_capacity, ptr(ws), nbytes, ptr(self.status), stream_ptr())
        return self

    @classmethod
    def from_topk(cls, topk_idx, topk_w, N, D, H, save_percent=0.0):
        M, K = topk_idx.shape
        return cls(M, N, K, D, H, topk_idx.device, save_percent).build(topk_idx, topk_w)

    @classmethod
    def from_mask(cls, mask_NM, s_NM, K, D, H, save_percent=0.0):
        """Compact an external router's dense mask_NM (int32, any strides) and s_NM (fp32, any strides)."""
        N, M = mask_NM.shape
        if mask_NM.dtype != torch.int32:
            mask_NM = mask_NM.to(torch.int32)
        if s_NM.dtype != torch.float32:
            s_NM = s_NM.to(torch.float32)
        dev = mask_NM.device
        plan = cls(M, N, K, D, H, dev, save_percent)
        topk_idx = torch.empty((M, K), dtype=torch.int32, device=dev)
        topk_w = torch.empty((M, K), dtype=torch.float32, device=dev)
        _call("momoe_topk_from_mask", 1, lib.momoe_topk_from_mask, ptr(mask_NM), mask_NM.stride(0), mask_NM.stride(1), ptr(s_NM),
                                       s_NM.stride(0), s_NM.stride(1), M, N, K, ptr(topk_idx), ptr(topk_w),
                                       ptr(plan.status), stream_ptr())
        return plan.build(topk_idx, topk_w)


def route_topk(logits_MN, biases_N, K, Ks, dense=True, normalisers=False):
    """Router after the gate GEMM.  Returns (topk_idx, topk_w, dict or None): the dict holds the dense outputs
    (dense=True) or only Ng_M / Ks_M (normalisers=True)."""
    _lib.require_cuda(logits_MN, biases_N)
    M, N = logits_MN.shape
    dev = logits_MN.device
    logits_MN = logits_MN.contiguous()
    biases_N = biases_N.to(device=dev, dtype=torch.float32).contiguous()
    topk_idx = torch.empty((M, K), dtype=torch.int32, device=dev)
    topk_w = torch.empty((M, K), dtype=torch.float32, device=dev)
    d = None
    if dense:
        d = dict(mask_NM=torch.empty((N, M), dtype=torch.int32, device=dev),
                 s_MN=torch.empty((M, N), dtype=torch.float32, device=dev),
                 s_postsoft_MN=torch.empty((M, N), dtype=torch.float32, device=dev),
                 Ng_M=torch.empty(M, dtype=torch.float32, device=dev),
                 Ks_M=torch.empty(M, dtype=torch.float32, device=dev))
    elif normalisers:
        d = dict(Ng_M=torch.empty(M, dtype=torch.float32, device=dev),
                 Ks_M=torch.empty(M, dtype=torch.float32, device=dev))
    _call("momoe_route_topk", 1, lib.momoe_route_topk, ptr(logits_MN), ptr(biases_N), M, N, K, Ks, ptr(topk_idx), ptr(topk_w),
                               ptr(d["mask_NM"]) if dense else None, ptr(d["s_MN"]) if dense else None,
                               ptr(d["s_postsoft_MN"]) if dense else None, ptr(d["Ng_M"]) if d else None,
                               ptr(d["Ks_M"]) if d else None, stream_ptr())
    return topk_idx, topk_w, d


def gather_rows(plan, src, cols):
    dst = torch.empty((plan.rows_capacity, cols), dtype=torch.bfloat16, device=src.device)
    _call("momoe_gather_rows", 1, lib.momoe_gather_rows, plan.ref, ptr(src), cols, ptr(dst), stream_ptr())
    return dst


def combine_rows(plan, src_sorted, cols):
    dst = torch.empty((plan.M, cols), dtype=torch.bfloat16, device=src_sorted.device)
    _call("momoe_combine_rows", 1, lib.momoe_combine_rows, plan.ref, ptr(src_sorted), cols, ptr(dst), stream_ptr())
    return dst


# MOMOE_B200_FUSED_GATHER=1 folds the row gathers into the grouped GEMMs (TMA row-gather loads of the token-major x and
# upstream gradient driven by the plan's row table): no expert-major copy of either is written or read, which saves
# two [rows, D] buffers and 1.1 GB of memory traffic per step on the headline layer.  Off by default: a row-gather load
# moves 4 rows x 128 bytes in about 75 SM cycles, four times slower than a tiled load, and the GEMMs then wait for
# their operands (0.93 -> 2.5 ms for the up projection).
FUSED_GATHER = os.environ.get("MOMOE_B200_FUSED_GATHER", "0") == "1"

# Forward-only calls with at most this many rows per expert on average take the weight-streaming kernels
# (momoe_up_swiglu_decode / momoe_down_scale_decode) instead of the 256-row tile kernels.
DECODE_MAX_AVG_ROWS = int(os.environ.get("MOMOE_B200_DECODE_ROWS", "16"))


def experts_forward(plan, x_MD, W1, W2, inference=False):
    """x_MD bf16 [M,D] contiguous; W1 bf16 [N,D,2H], W2 bf16 [N,H,D] contiguous.
    Returns y_MD bf16 and the (a, b) buffers saved for the backward pass (None when nothing is saved).
    inference=True: no backward pass will follow; small batches then use the weight-streaming kernels."""
    dev = x_MD.device
    D, H = plan.D, plan.H
    bf = dict(dtype=torch.bfloat16, device=dev)
    h = torch.empty((plan.rows_capacity, H), **bf)
    y_sorted = torch.empty((plan.rows_capacity, D), **bf)
    if inference and plan.Msum <= DECODE_MAX_AVG_ROWS * plan.N:
        x_sorted = gather_rows(plan, x_MD, D)
        _call("momoe_up_swiglu_decode", 1, lib.momoe_up_swiglu_decode, plan.ref, ptr(x_sorted), ptr(W1), ptr(h),
              stream_ptr())
        _call("momoe_down_scale_decode", 1, lib.momoe_down_scale_decode, plan.ref, ptr(h), ptr(W2), ptr(y_sorted),
              stream_ptr())
        return combine_rows(plan, y_sorted, D), None, None
    a_save = b_save = None
    mode = 0
    if plan.saved_tile_capacity > 0:
        a_save = torch.empty((plan.saved_tile_capacity * TILE_M, H), **bf)
        b_save = torch.empty((plan.saved_tile_capacity * TILE_M, H), **bf)
        mode = 1
    if FUSED_GATHER:
        _call("momoe_up_swiglu", 1, lib.momoe_up_swiglu_tokens, plan.ref, ptr(x_MD), ptr(W1), ptr(h), ptr(a_save),
              ptr(b_save), mode, stream_ptr())
    else:
        x_sorted = gather_rows(plan, x_MD, D)
        _call("momoe_up_swiglu", 1, lib.momoe_up_swiglu, plan.ref, ptr(x_sorted), ptr(W1), ptr(h), ptr(a_save),
              ptr(b_save), mode, stream_ptr())
        del x_sorted
    _call("momoe_down_scale", 1, lib.momoe_down_scale, plan.ref, ptr(h), ptr(W2), ptr(y_sorted), stream_ptr())
    return combine_rows(plan, y_sorted, D), a_save, b_save


def experts_backward(plan, g_MD, x_MD, W1, W2, a_save, b_save, need_gs_dense=True):
    """Returns G_x bf16 [M,D], G_W1 bf16, G_W2 bf16, G_s (dense fp32 [N,M] or per-row partial sums)."""
    dev = x_MD.device
    D, H, N = plan.D, plan.H, plan.N
    bf = dict(dtype=torch.bfloat16, device=dev)
    fused = FUSED_GATHER
    if fused:
        g_src, x_src = g_MD, x_MD            # token-major: the GEMMs fetch rows through the plan's row table
        up, dgrad2 = lib.momoe_up_swiglu_tokens, lib.momoe_dgrad2_swiglu_bwd_tokens
    else:
        g_src = gather_rows(plan, g_MD, D)
        x_src = gather_rows(plan, x_MD, D)
        up, dgrad2 = lib.momoe_up_swiglu, lib.momoe_dgrad2_swiglu_bwd
    a_rec = b_rec = None
    if plan.recomp_tile_capacity > 0:
        a_rec = torch.empty((plan.recomp_tile_capacity * TILE_M, H), **bf)
        b_rec = torch.empty((plan.recomp_tile_capacity * TILE_M, H), **bf)
        _call("momoe_up_swiglu (recompute)", 1, up, plan.ref, ptr(x_src), ptr(W1), None, ptr(a_rec), ptr(b_rec), 2,
              stream_ptr())
    n_part = 2 * ((H + 255) // 256)   # two partial sums per 256-column block (momoe_dgrad2_swiglu_bwd)
    gz = torch.empty((plan.rows_capacity, 2 * H), **bf)
    hs = torch.empty((plan.rows_capacity, H), **bf)
    gs_part = torch.empty((plan.rows_capacity, n_part), dtype=torch.float32, device=dev)
    _call("momoe_dgrad2_swiglu_bwd", 1, dgrad2, plan.ref, ptr(g_src), ptr(W2), ptr(a_save), ptr(b_save), ptr(a_rec),
          ptr(b_rec), ptr(gz), ptr(hs), ptr(gs_part), stream_ptr())
    del a_rec, b_rec
    G_W2 = torch.empty_like(W2)
    G_W1 = torch.empty_like(W1)
    if fused:
        _call("momoe_wgrad (W2)", 1, lib.momoe_wgrad_tokens, plan.ref, ptr(hs), H, 0, ptr(g_src), D, 1, ptr(G_W2),
              stream_ptr())
        _call("momoe_wgrad (W1)", 1, lib.momoe_wgrad_tokens, plan.ref, ptr(x_src), D, 1, ptr(gz), 2 * H, 0, ptr(G_W1),
              stream_ptr())
        del hs
        gx_sorted = torch.empty((plan.rows_capacity, D), **bf)
    else:
        _call("momoe_wgrad (W2)", 1, lib.momoe_wgrad, plan.ref, ptr(hs), H, ptr(g_src), D, ptr(G_W2), stream_ptr())
        _call("momoe_wgrad (W1)", 1, lib.momoe_wgrad, plan.ref, ptr(x_src), D, ptr(gz), 2 * H, ptr(G_W1), stream_ptr())
        gx_sorted = g_src  # the gathered upstream gradient is dead after the W2 gradient; reuse its buffer
    _call("momoe_dgrad1", 1, lib.momoe_dgrad1, plan.ref, ptr(gz), ptr(W1), ptr(gx_sorted), stream_ptr())
    G_x = combine_rows(plan, gx_sorted, D)
    if need_gs_dense:
        G_s = torch.empty((N, plan.M), dtype=torch.float32, device=dev)
        _call("momoe_scatter_gs", 1, lib.momoe_scatter_gs, plan.ref, ptr(gs_part), n_part, ptr(G_s), stream_ptr())
    else:
        G_s = gs_part
    return G_x, G_W1, G_W2, G_s


def router_backward(G_s_NM, s_postsoft_MN, s_MN, Ng_M, Ks_M, mask_NM, Ks):
    N, M = G_s_NM.shape
    if G_s_NM.dtype != torch.float32:
        G_s_NM = G_s_NM.to(torch.float32)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=G_s_NM.device)
    _call("momoe_router_backward", 1, lib.momoe_router_backward, ptr(G_s_NM), G_s_NM.stride(0), G_s_NM.stride(1), ptr(s_postsoft_MN), ptr(s_MN),
                                    ptr(Ng_M), ptr(Ks_M), ptr(mask_NM), M, N, Ks, ptr(out), stream_ptr())
    return out


def router_backward_compact(plan, gs_part, Ng_M, Ks_M, Ks):
    """Gradient of the gate logits (bf16 [M,N]) straight from the experts' per-row partial sums."""
    out = torch.empty((plan.M, plan.N), dtype=torch.bfloat16, device=gs_part.device)
    _call("momoe_router_backward_compact", 1, lib.momoe_router_backward_compact, plan.ref, ptr(gs_part),
          gs_part.shape[1], ptr(plan.topk_idx), ptr(plan.topk_w), ptr(Ng_M), ptr(Ks_M), Ks, ptr(out), stream_ptr())
    return out


def router_backward_from_topk_grad(G_w_MK, topk_idx, topk_w, Ng_M, Ks_M, N, Ks):
    """Gradient of the gate logits (bf16 [M,N]) from dL/d topk_w (fp32 [M,K])."""
    M, K = topk_idx.shape
    G_w_MK = G_w_MK.to(torch.float32).contiguous()
    out = torch.empty((M, N), dtype=torch.bfloat16, device=topk_idx.device)
    c = _lib.Plan(M=M, N=N, K=K, D=0, H=0, reserved=0, rows_capacity=0, sched=0, tile_expert=0, pad_off=0,
                  row_token=0, row_weight=0, pos_MK=0, status=0, pair_info=0)
    _call("momoe_router_backward_compact", 1, lib.momoe_router_backward_compact, C.byref(c), ptr(G_w_MK), 1,
          ptr(topk_idx), ptr(topk_w), ptr(Ng_M), ptr(Ks_M), Ks, ptr(out), stream_ptr())
    return out


def bias_update_(biases_N, sizes_N, Ks, c_avg, rate):
    """In-place aux-loss-free bias update (one kernel instead of the reference's three torch ops)."""
    N = biases_N.shape[0]
    sizes_N = sizes_N.to(device=biases_N.device, dtype=torch.int64)
    _call("momoe_bias_update", 1, lib.momoe_bias_update, ptr(biases_N), ptr(sizes_N), N, Ks, float(c_avg), float(rate),
          stream_ptr())
