"""Expert parallelism for the MoMoE layer (the reference has none; its README lists it as unsupported).

Rank r of an R-rank group owns the contiguous expert block [r*N/R, (r+1)*N/R) and keeps its own tokens
(data parallel).  Two transports:

* ``"peer"`` (default inside one NVLink node): buffers every rank can address (torch symmetric memory).  The
  per-expert counts are exchanged by peer stores and a flag hand-shake, every rank derives the whole dispatch plan on
  the device, token rows are stored straight into the owner's padded expert-major buffer (gather + send in one
  kernel) and results are summed straight out of the owners' buffers (receive + reduce in one kernel).  The host
  never synchronises and nothing is staged.
* ``"nccl"``: all-gather of counts (one host synchronisation for the split sizes), all-to-all-v of rows, local
  re-sort.  Works wherever NCCL does; `DispatchMeta` holds its index arithmetic (device-agnostic torch ops, tested
  with CPU ranks).

Backward mirrors forward with the upstream gradient.  Payload always lands in the owner's own memory before the
grouped GEMMs read it; no TMA load ever addresses a peer.
"""
import ctypes as C
import os
import weakref

import torch
import torch.distributed as dist
import torch.nn as nn

from . import ops
from .momoe import _CHECK
from .topk_router import CompactRouterFunction, TopKRouter


class DispatchMeta:
    """Index arithmetic of one dispatch, built from this rank's routing and the all-gathered counts.

    sizes_RN  int64 [R, N]  tokens rank s routes to global expert e (row s = rank s's `sizes_N`)
    idx, which int32 [M*K]  this rank's expert-major permutation (token of each row, slot of each row)
    """

    def __init__(self, sizes_RN, idx, which, rank, M, K):
        R, N = sizes_RN.shape
        assert N % R == 0, "experts must divide evenly across ranks"
        self.R, self.N, self.Nl, self.rank, self.M, self.K = R, N, N // R, rank, M, K
        per_block = sizes_RN.view(R, R, self.Nl).sum(-1)               # [source, destination]
        self.send_splits = per_block[rank].tolist()                    # rows this rank sends to each rank
        self.recv_splits = per_block[:, rank].tolist()                 # rows this rank receives from each rank
        self.n_send = int(sum(self.send_splits))
        self.n_recv = int(sum(self.recv_splits))
        assert self.n_send == M * K
        dev = idx.device
        # local expert (0..Nl-1) of every received row: source-major, inside a source expert-major
        mine = sizes_RN[:, rank * self.Nl:(rank + 1) * self.Nl].reshape(-1).to(dev)
        self.recv_expert = torch.arange(self.Nl, device=dev, dtype=torch.int32).repeat(R).repeat_interleave(
            mine, output_size=self.n_recv)
        # row of token m's k-th expert in the (unpadded) send order
        self.pos_unpadded = torch.empty(M * K, dtype=torch.int32, device=dev)
        self.pos_unpadded[idx.long() * K + which.long()] = torch.arange(M * K, dtype=torch.int32, device=dev)
        # global expert of every sent row (for the dense G_s the router backward consumes)
        self.send_expert = torch.arange(N, device=dev).repeat_interleave(sizes_RN[rank].to(dev), output_size=M * K)
        self.global_sizes = sizes_RN.sum(0)


def exchange(t_send, send_splits, recv_splits, group):
    """all-to-all-v over rows of a [rows, ...] tensor."""
    out = t_send.new_empty((int(sum(recv_splits)),) + tuple(t_send.shape[1:]))
    dist.all_to_all_single(out, t_send.contiguous(), recv_splits, send_splits, group=group)
    return out


def gather_counts(sizes_N, group):
    R = dist.get_world_size(group)
    out = torch.empty(R * sizes_N.numel(), dtype=sizes_N.dtype, device=sizes_N.device)
    dist.all_gather_into_tensor(out, sizes_N.contiguous(), group=group)
    return out.view(R, sizes_N.numel()).cpu()   # host copy: NCCL split sizes are host integers


class _Rows:
    """Row movers on the device through the C ABI, addressed with ad-hoc row tables."""

    @staticmethod
    def gather(src, row_index, n_rows):
        """dst[r] = src[row_index[r]] for r < n_rows (bf16 rows)."""
        from . import _lib, ops
        cols = src.shape[1]
        dst = torch.empty((n_rows, cols), dtype=torch.bfloat16, device=src.device)
        if n_rows == 0:
            return dst
        sched = torch.tensor([0, 0, n_rows, 0, 0, 0, 0, 0], dtype=torch.int32, device=src.device)
        plan = _lib.Plan(M=1, N=1, K=1, D=cols, H=8, reserved=0, rows_capacity=128, sched=sched.data_ptr(),
                         tile_expert=0, pad_off=0, row_token=row_index.data_ptr(), row_weight=0, pos_MK=0, status=0)
        ops._call("momoe_gather_rows", 1, _lib.lib.momoe_gather_rows, C.byref(plan), _lib.ptr(src), cols,
                  _lib.ptr(dst), _lib.stream_ptr())
        return dst

    @staticmethod
    def combine(src, pos_MK, M, K):
        """dst[m] = bf16(sum_k src[pos_MK[m, k]])."""
        from . import _lib, ops
        cols = src.shape[1]
        dst = torch.empty((M, cols), dtype=torch.bfloat16, device=src.device)
        plan = _lib.Plan(M=M, N=1, K=K, D=cols, H=8, reserved=0, rows_capacity=128, sched=0, tile_expert=0, pad_off=0,
                         row_token=0, row_weight=0, pos_MK=pos_MK.data_ptr(), status=0)
        ops._call("momoe_combine_rows", 1, _lib.lib.momoe_combine_rows, C.byref(plan), _lib.ptr(src), cols,
                  _lib.ptr(dst), _lib.stream_ptr())
        return dst


class ExpertParallelFunction(torch.autograd.Function):
    """Forward / backward of the expert computation with dispatch and combine over the process group."""

    @staticmethod
    def forward(ctx, x_BSD, W1_local, W2_local, mask_NM, s_NM, topk_idx, topk_w, K, save_percent, group):
        from . import ops
        B, S, D = x_BSD.shape
        M = B * S
        dev = W1_local.device
        Nl, H, _ = W2_local.shape
        R = dist.get_world_size(group)
        rank = dist.get_rank(group)
        N = Nl * R
        x_MD = x_BSD.reshape(M, D).to(device=dev, dtype=torch.bfloat16).contiguous()
        W1 = W1_local.detach().to(torch.bfloat16).contiguous()
        W2 = W2_local.detach().to(torch.bfloat16).contiguous()
        with torch.cuda.device(dev):
            home = ops.RoutingPlan.from_topk(topk_idx, topk_w, N, D, H, 0.0)     # permutation over all N experts
            sizes_RN = gather_counts(home.sizes, group)
            meta = DispatchMeta(sizes_RN, home.idx, home.which, rank, M, K)
            x_send = _Rows.gather(x_MD, home.idx, meta.n_send)
            w_send = topk_w.reshape(-1)[(home.idx.long() * K + home.which.long())].contiguous()
            x_recv = exchange(x_send, meta.send_splits, meta.recv_splits, group)
            w_recv = exchange(w_send, meta.send_splits, meta.recv_splits, group)
            del x_send
            # the received rows are this rank's "tokens", each routed to exactly one local expert
            if meta.n_recv > 0:
                local = ops.RoutingPlan.from_topk(meta.recv_expert.view(-1, 1), w_recv.view(-1, 1), Nl, D, H,
                                                  save_percent)
                y_recv, a_save, b_save = ops.experts_forward(local, x_recv, W1, W2)
            else:
                local, a_save, b_save = None, None, None
                y_recv = x_recv
            y_back = exchange(y_recv, meta.recv_splits, meta.send_splits, group)
            y_MD = _Rows.combine(y_back, meta.pos_unpadded, M, K)
        ctx.group, ctx.meta, ctx.home, ctx.local = group, meta, home, local
        ctx.shape = (B, S, D)
        ctx.dims = (N, Nl, H, K)
        ctx.in_devices = (x_BSD.device, s_NM.device)
        ctx.has_ab = a_save is not None
        saved = [x_recv, W1, W2] + ([a_save, b_save] if ctx.has_ab else [])
        ctx.save_for_backward(*saved)
        sizes_global = meta.global_sizes.to(dev)
        ctx.mark_non_differentiable(sizes_global)
        return y_MD.reshape(B, S, D).to(x_BSD.device), sizes_global

    @staticmethod
    def backward(ctx, G_y_BSD, _):
        from . import ops
        saved = ctx.saved_tensors
        x_recv, W1, W2 = saved[:3]
        a_save, b_save = (saved[3], saved[4]) if ctx.has_ab else (None, None)
        B, S, D = ctx.shape
        N, Nl, H, K = ctx.dims
        M = B * S
        meta, home, local, group = ctx.meta, ctx.home, ctx.local, ctx.group
        dev = W1.device
        g_MD = G_y_BSD.reshape(M, D).to(device=dev, dtype=torch.bfloat16).contiguous()
        with torch.cuda.device(dev):
            g_send = _Rows.gather(g_MD, home.idx, meta.n_send)
            g_recv = exchange(g_send, meta.send_splits, meta.recv_splits, group)
            del g_send
            if local is not None:
                gx_recv, G_W1, G_W2, gs_part = ops.experts_backward(local, g_recv, x_recv, W1, W2, a_save, b_save,
                                                                    need_gs_dense=False)
                gs_recv = gs_part.sum(-1)[local.pos.long()].contiguous()      # K = 1: pos[j] is row j's padded row
            else:
                gx_recv = g_recv
                G_W1, G_W2 = torch.zeros_like(W1), torch.zeros_like(W2)
                gs_recv = torch.empty(0, dtype=torch.float32, device=dev)
            gx_back = exchange(gx_recv, meta.recv_splits, meta.send_splits, group)
            gs_back = exchange(gs_recv, meta.recv_splits, meta.send_splits, group)
            G_x = _Rows.combine(gx_back, meta.pos_unpadded, M, K)
            G_s = torch.zeros((N, M), dtype=torch.float32, device=dev)
            G_s[meta.send_expert, home.idx.long()] = gs_back
        x_dev, s_dev = ctx.in_devices
        return (G_x.reshape(B, S, D).to(x_dev), G_W1, G_W2, None, G_s.to(s_dev), None, None, None, None, None)


class PeerBuffers:
    """Symmetric (peer-addressable) buffers of one expert-parallel layer and the epoch counter of its hand-shakes."""

    def __init__(self, group, device, N, D, cap_rows):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.cap_rows = cap_rows
        self.epoch = 0
        self._keep = []
        self.max_tokens = 0        # tokens per rank the buffers were sized for (set by the layer)
        self.forward_chunks = None  # 1: transfers and GEMMs of a forward pass in sequence; 2: in two overlapping halves;
                                    # None: 2 for passes that move at least 16 MiB of rows per rank
        self._step = 0             # forward passes started
        self._pending = 0          # step whose backward pass has not run yet (0: none)

        def alloc(shape, dtype):
            t = symm_mem.empty(shape, dtype=dtype, device=device)
            t.zero_()
            h = symm_mem.rendezvous(t, group)
            self._keep.append(h)
            arr = (C.c_void_p * self.world)(*[C.c_void_p(int(p)) for p in h.buffer_ptrs])
            return t, arr

        self.rows_x, self.p_rows_x = alloc((cap_rows, D), torch.bfloat16)     # dispatched activations (kept for backward)
        self.rows_y, self.p_rows_y = alloc((cap_rows, D), torch.bfloat16)     # expert outputs / input gradients
        self.rows_g, self.p_rows_g = alloc((cap_rows, D), torch.bfloat16)     # dispatched upstream gradient
        self.row_w, self.p_row_w = alloc((cap_rows,), torch.float32)          # routing weight of each received row
        self.row_gs, self.p_row_gs = alloc((cap_rows,), torch.float32)        # dL/ds of each received row
        self.counts, self.p_counts = alloc((self.world * N,), torch.int32)
        # Two hand-shake channels of 8 flag words each, with epoch counters of their own: hand-shakes queued on the
        # transfer stream must not be satisfied by (or satisfy) the ones queued on the main stream in the same pass.
        self.flags, self.p_flags = alloc((16,), torch.int32)
        self.p_flags_b = (C.c_void_p * self.world)(*[C.c_void_p(int(p) + 32) for p in self._keep[-1].buffer_ptrs])
        self.epoch_b = 0
        self.comm_stream = torch.cuda.Stream(device=device)
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        torch.cuda.synchronize(device)
        dist.barrier(group)     # every rank's buffers are zeroed before anybody signals

    def next_epoch(self):
        self.epoch += 1
        return self.epoch

    def next_epoch_b(self):
        self.epoch_b += 1
        return self.epoch_b

    # One set of buffers serves one step at a time: `rows_x` / `row_w` written by a forward pass are read again by its
    # backward pass, and `rows_y` / `rows_g` are reused by both.  A second forward pass before that backward pass
    # (pipeline micro-batches, activation checkpointing, an evaluation pass in between) would silently overwrite them,
    # so it is refused instead.
    def begin_step(self, needs_backward):
        if self._pending:
            raise RuntimeError(
                "ExpertParallelMoE (peer transport): forward called while the backward pass of the previous forward is "
                "still outstanding; its peer buffers hold one step at a time.  Run the backward pass first, wrap "
                "passes that need no gradient in torch.no_grad(), drop the previous output, or use transport='nccl'.")
        self._step += 1
        if needs_backward:
            self._pending = self._step
        return self._step

    def end_step(self, step):
        if self._pending == step:
            self._pending = 0


class _StepToken:
    """Lifetime marker of one forward pass's autograd node."""


class PeerExpertParallelFunction(torch.autograd.Function):
    """Expert computation with dispatch / combine over peer memory (see the module docstring)."""

    @staticmethod
    def forward(ctx, x_BSD, W1_local, W2_local, topk_idx, topk_w, K, save_percent, bufs):
        from . import _lib, ops
        lib, ptr, st = _lib.lib, _lib.ptr, _lib.stream_ptr
        B, S, D = x_BSD.shape
        M = B * S
        dev = W1_local.device
        Nl, H, _ = W2_local.shape
        R, rank = bufs.world, bufs.rank
        N = Nl * R
        cap = bufs.cap_rows
        i32 = dict(dtype=torch.int32, device=dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        x_MD = x_BSD.reshape(M, D).to(device=dev, dtype=torch.bfloat16).contiguous()
        W1 = W1_local.detach().to(torch.bfloat16).contiguous()
        W2 = W2_local.detach().to(torch.bfloat16).contiguous()
        step = bufs.begin_step(any(ctx.needs_input_grad))
        ctx.step = step
        ctx.step_token = _StepToken()      # dies with the autograd graph: an output dropped without backward frees the buffers
        weakref.finalize(ctx.step_token, bufs.end_step, step)
        # Two halves of the local experts when the pass is large enough to be bound by the transfers rather than by
        # launch latency: the rows of the second half travel while the GEMMs work on the first half, and the results
        # of the first half travel back while the GEMMs work on the second.
        chunks = bufs.forward_chunks
        if chunks is None:
            # decided from the token count the buffers were sized for, which is the same number on every rank (ranks
            # may bring different numbers of tokens, but all of them must take the same sequence of hand-shakes)
            chunks = 2 if max(bufs.max_tokens, 1) * K * D * 2 >= (16 << 20) else 1
        split = Nl // 2 if (chunks == 2 and Nl >= 2) else 0
        with torch.cuda.device(dev):
            home = ops.RoutingPlan.from_topk(topk_idx, topk_w, N, D, H, 0.0)
            status = home.status
            ops._call("momoe_ep_publish_counts", 1, lib.momoe_ep_publish_counts, ptr(home.sizes), N, bufs.p_counts,
                      bufs.p_flags, R, rank, bufs.next_epoch(), ptr(status), st())
            tile_cap = cap // ops.TILE_M
            dst_base = torch.empty(N, **i32)
            sizes_global = torch.empty(N, dtype=torch.int64, device=dev)
            local_count = torch.empty(Nl, **i32)
            pad_off = torch.empty(Nl + 1, **i32)
            tile_expert = torch.empty(tile_cap, **i32)
            pair_info = torch.empty(tile_cap, **i32)
            sched = torch.empty(8, **i32)
            remote_row = torch.empty(home.rows_capacity, **i32)

            def local_plan(sched_t, sched_off, pair_t, pair_off):
                return _lib.Plan(M=1, N=Nl, K=1, D=D, H=H, reserved=0, rows_capacity=cap,
                                 sched=sched_t.data_ptr() + 4 * sched_off, tile_expert=tile_expert.data_ptr(),
                                 pad_off=pad_off.data_ptr(), row_token=0, row_weight=bufs.row_w.data_ptr(), pos_MK=0,
                                 status=status.data_ptr(), pair_info=pair_t.data_ptr() + 4 * pair_off)

            h = torch.empty((cap, H), **bf)
            a_save = b_save = None
            mode = 0
            if save_percent > 0:
                a_save = torch.empty((cap, H), **bf)
                b_save = torch.empty((cap, H), **bf)
                mode = 1
            y_MD = torch.empty((M, D), **bf)

            def gemms(plan_c):
                ops._call("momoe_up_swiglu", 1, lib.momoe_up_swiglu, C.byref(plan_c), ptr(bufs.rows_x), ptr(W1),
                          ptr(h), ptr(a_save), ptr(b_save), mode, st())
                ops._call("momoe_down_scale", 1, lib.momoe_down_scale, C.byref(plan_c), ptr(h), ptr(W2),
                          ptr(bufs.rows_y), st())

            if split == 0:
                ops._call("momoe_ep_plan", 1, lib.momoe_ep_plan, ptr(bufs.counts), R, rank, N, float(save_percent),
                          cap, ptr(dst_base), ptr(sizes_global), ptr(local_count), ptr(pad_off), ptr(tile_expert),
                          ptr(pair_info), ptr(sched), ptr(status), st())
                local = local_plan(sched, 0, pair_info, 0)
                ops._call("momoe_ep_dispatch_rows", 1, lib.momoe_ep_dispatch_rows, home.ref, ptr(x_MD), D,
                          ptr(dst_base), Nl, bufs.p_rows_x, bufs.p_row_w, ptr(remote_row), R, rank, ptr(local_count),
                          ptr(pad_off), 0, st())
                ops._call("momoe_ep_barrier", 1, lib.momoe_ep_barrier, bufs.p_flags, R, rank, bufs.next_epoch(),
                          ptr(status), st())
                # local experts on the received rows: already expert-major and padded
                gemms(local)
                ops._call("momoe_ep_barrier", 1, lib.momoe_ep_barrier, bufs.p_flags, R, rank, bufs.next_epoch(),
                          ptr(status), st())
                ops._call("momoe_ep_combine_rows", 1, lib.momoe_ep_combine_rows, home.ref, bufs.p_rows_y,
                          ptr(remote_row), Nl, D, ptr(y_MD), R, 0, st())
                parts = None
            else:
                pair_parts = torch.empty(2 * tile_cap, **i32)
                sched_parts = torch.empty(16, **i32)
                ops._call("momoe_ep_plan", 1, lib.momoe_ep_plan_split, ptr(bufs.counts), R, rank, N,
                          float(save_percent), cap, ptr(dst_base), ptr(sizes_global), ptr(local_count), ptr(pad_off),
                          ptr(tile_expert), ptr(pair_info), ptr(sched), split, ptr(pair_parts), ptr(sched_parts),
                          ptr(status), st())
                local = local_plan(sched, 0, pair_info, 0)
                part = [local_plan(sched_parts, 0, pair_parts, 0), local_plan(sched_parts, 8, pair_parts, tile_cap)]
                parts = (pair_parts, sched_parts)
                main = torch.cuda.current_stream()
                comm = bufs.comm_stream
                one_per_sm = bufs.sm_count
                ev = [torch.cuda.Event() for _ in range(4)]
                staged = torch.empty((home.rows_capacity, D), **bf)
                # rows of the first half of every rank's experts; everything else waits for them
                ops._call("momoe_ep_dispatch_rows", 1, lib.momoe_ep_dispatch_rows_range, home.ref, ptr(x_MD), D,
                          ptr(dst_base), Nl, bufs.p_rows_x, bufs.p_row_w, ptr(remote_row), R, rank, ptr(local_count),
                          ptr(pad_off), 0, split, 0, st())
                ev[0].record(main)
                ops._call("momoe_ep_barrier", 1, lib.momoe_ep_barrier, bufs.p_flags, R, rank, bufs.next_epoch(),
                          ptr(status), st())
                with torch.cuda.stream(comm):
                    # rows of the second half beside the GEMMs of the first half
                    comm.wait_event(ev[0])
                    ops._call("momoe_ep_dispatch_rows", 1, lib.momoe_ep_dispatch_rows_range, home.ref, ptr(x_MD), D,
                              ptr(dst_base), Nl, bufs.p_rows_x, bufs.p_row_w, ptr(remote_row), R, rank,
                              ptr(local_count), ptr(pad_off), split, Nl, one_per_sm, st())
                    ops._call("momoe_ep_barrier", 1, lib.momoe_ep_barrier, bufs.p_flags_b, R, rank,
                              bufs.next_epoch_b(), ptr(status), st())
                    ev[1].record(comm)
                gemms(part[0])
                ev[2].record(main)
                with torch.cuda.stream(comm):
                    # results of the first half come home beside the GEMMs of the second half
                    comm.wait_event(ev[2])
                    ops._call("momoe_ep_barrier", 1, lib.momoe_ep_barrier, bufs.p_flags_b, R, rank,
                              bufs.next_epoch_b(), ptr(status), st())
                    ops._call("momoe_ep_pull_rows", 1, lib.momoe_ep_pull_rows, home.ref, bufs.p_rows_y,
                              ptr(remote_row), Nl, D, ptr(staged), R, rank, 0, split, one_per_sm, st())
                    ev[3].record(comm)
                main.wait_event(ev[1])
                gemms(part[1])
                ops._call("momoe_ep_barrier", 1, lib.momoe_ep_barrier, bufs.p_flags, R, rank, bufs.next_epoch(),
                          ptr(status), st())
                main.wait_event(ev[3])
                ops._call("momoe_ep_combine_rows", 1, lib.momoe_ep_combine_rows_staged, home.ref, bufs.p_rows_y,
                          ptr(remote_row), Nl, D, ptr(y_MD), R, ptr(staged), 0, split, 0, st())
                staged.record_stream(comm)
                x_MD.record_stream(comm)
                del staged
            del h
        ctx.bufs, ctx.home, ctx.local = bufs, home, local
        ctx.keep = (dst_base, local_count, pad_off, tile_expert, pair_info, sched, remote_row)
        ctx.parts = parts      # tables the GEMMs of the two halves read: alive until the kernels have run
        ctx.shape = (B, S, D)
        ctx.dims = (N, Nl, H, K)
        ctx.save_percent = save_percent
        ctx.in_devices = (x_BSD.device, topk_w.device)
        ctx.has_ab = a_save is not None
        ctx.save_for_backward(*([W1, W2] + ([a_save, b_save] if ctx.has_ab else [])))
        ctx.mark_non_differentiable(sizes_global)
        ops.status_post(dev)
        if _CHECK:
            ops.check_status(dev)
        return y_MD.reshape(B, S, D).to(x_BSD.device), sizes_global

    @staticmethod
    def backward(ctx, G_y_BSD, _):
        from . import _lib, ops
        lib, ptr, st = _lib.lib, _lib.ptr, _lib.stream_ptr
        saved = ctx.saved_tensors
        W1, W2 = saved[:2]
        a_save, b_save = (saved[2], saved[3]) if ctx.has_ab else (None, None)
        B, S, D = ctx.shape
        N, Nl, H, K = ctx.dims
        M = B * S
        bufs, home, local = ctx.bufs, ctx.home, ctx.local
        dst_base, local_count, pad_off, tile_expert, pair_info, sched, remote_row = ctx.keep
        R, rank, cap = bufs.world, bufs.rank, bufs.cap_rows
        dev = W1.device
        bf = dict(dtype=torch.bfloat16, device=dev)
        status = home.status
        g_MD = G_y_BSD.reshape(M, D).to(device=dev, dtype=torch.bfloat16).contiguous()
        with torch.cuda.device(dev):
            # Two streams.  The transfers (peer stores / loads, one small block per SM) run on `comm` while grouped
            # GEMMs that do not depend on them run on the main stream on the same SMs:
            #   dispatch of the upstream gradient  ||  recomputation of a,b (needs only the rows kept from forward)
            #   combine of the input gradient      ||  the two weight-gradient GEMMs
            main = torch.cuda.current_stream()
            comm = bufs.comm_stream
            one_per_sm = bufs.sm_count
            ev = [torch.cuda.Event() for _ in range(4)]
            ev[0].record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(ev[0])
                ops._call("momoe_ep_dispatch_rows", 1, lib.momoe_ep_dispatch_rows, home.ref, ptr(g_MD), D,
                          ptr(dst_base), Nl, bufs.p_rows_g, None, None, R, rank, ptr(local_count), ptr(pad_off),
                          one_per_sm, st())
                ops._call("momoe_ep_barrier", 1, lib.momoe_ep_barrier, bufs.p_flags, R, rank, bufs.next_epoch(),
                          ptr(status), st())
                ev[1].record(comm)
            lp = C.byref(local)
            # Tiles that do not lie entirely below the save boundary are recomputed; even at save_percent = 100 the
            # last partial tile of an expert can be one of them, so the pass always runs (it skips saved tiles).
            rec_tiles = min(cap // ops.TILE_M,
                            int(cap * (100.0 - ctx.save_percent) / 100.0) // ops.TILE_M + Nl + 1)
            a_rec = torch.empty((rec_tiles * ops.TILE_M, H), **bf)
            b_rec = torch.empty((rec_tiles * ops.TILE_M, H), **bf)
            ops._call("momoe_up_swiglu (recompute)", 1, lib.momoe_up_swiglu, lp, ptr(bufs.rows_x), ptr(W1), None,
                      ptr(a_rec), ptr(b_rec), 2, st())
            main.wait_event(ev[1])
            n_part = 2 * ((H + 255) // 256)
            gz = torch.empty((cap, 2 * H), **bf)
            hs = torch.empty((cap, H), **bf)
            gs_part = torch.empty((cap, n_part), dtype=torch.float32, device=dev)
            ops._call("momoe_dgrad2_swiglu_bwd", 1, lib.momoe_dgrad2_swiglu_bwd, lp, ptr(bufs.rows_g), ptr(W2),
                      ptr(a_save), ptr(b_save), ptr(a_rec), ptr(b_rec), ptr(gz), ptr(hs), ptr(gs_part), st())
            ops._call("momoe_dgrad1", 1, lib.momoe_dgrad1, lp, ptr(gz), ptr(W1), ptr(bufs.rows_y), st())
            ops._call("momoe_ep_reduce_gs", 1, lib.momoe_ep_reduce_gs, ptr(gs_part), n_part, ptr(sched),
                      ptr(bufs.row_gs), st())
            ev[2].record(main)
            G_x = torch.empty((M, D), **bf)
            G_w = torch.empty((M, K), dtype=torch.float32, device=dev)
            with torch.cuda.stream(comm):
                comm.wait_event(ev[2])
                ops._call("momoe_ep_barrier", 1, lib.momoe_ep_barrier, bufs.p_flags, R, rank, bufs.next_epoch(),
                          ptr(status), st())
                ops._call("momoe_ep_combine_rows", 1, lib.momoe_ep_combine_rows, home.ref, bufs.p_rows_y,
                          ptr(remote_row), Nl, D, ptr(G_x), R, one_per_sm, st())
                ops._call("momoe_ep_pull_gs_compact", 1, lib.momoe_ep_pull_gs_compact, home.ref, bufs.p_row_gs,
                          ptr(remote_row), Nl, ptr(G_w), R, st())
                ev[3].record(comm)
            G_W2 = torch.empty_like(W2)
            ops._call("momoe_wgrad (W2)", 1, lib.momoe_wgrad, lp, ptr(hs), H, ptr(bufs.rows_g), D, ptr(G_W2), st())
            G_W1 = torch.empty_like(W1)
            ops._call("momoe_wgrad (W1)", 1, lib.momoe_wgrad, lp, ptr(bufs.rows_x), D, ptr(gz), 2 * H, ptr(G_W1), st())
            main.wait_event(ev[3])
        bufs.end_step(ctx.step)
        ops.status_post(dev)
        if _CHECK:
            ops.check_status(dev)
        x_dev, w_dev = ctx.in_devices
        return (G_x.reshape(B, S, D).to(x_dev), G_W1, G_W2, None, G_w.to(w_dev), None, None, None)


class _ExpertBlock(nn.Module):
    """This rank's block of N/R experts.  The layer names it `momoe`, so parameter keys read `momoe.Wl1_ND2H` /
    `momoe.Wl2_NHD` exactly as in the single-GPU `MoE` (momoe/sample_moe.py:48-55 of the reference)."""

    def __init__(self, Wl1_ND2H, Wl2_NHD):
        super().__init__()
        self.Wl1_ND2H = nn.Parameter(Wl1_ND2H.clone().detach().to(torch.bfloat16), requires_grad=True)
        self.Wl2_NHD = nn.Parameter(Wl2_NHD.clone().detach().to(torch.bfloat16), requires_grad=True)


class ExpertParallelMoE(nn.Module):
    """`MoE` with the experts sharded over a process group: same forward signature and bias update; the router is
    replicated, `momoe.Wl1_ND2H` / `momoe.Wl2_NHD` hold this rank's block of N/R experts, and `tokens_per_expert_N`
    (which drives the bias update) is the global count summed over ranks.

    Checkpoints keep the single-GPU layout and key names (`router.Wg_DN`, `momoe.Wl1_ND2H`, `momoe.Wl2_NHD`,
    `biases_N`; momoe/sample_moe.py:39-57, momoe/momoe.py:947-955 of the reference): `load_state_dict` accepts a
    checkpoint of the single-GPU layer (every rank keeps its block of the `[N, ...]` tensors; a checkpoint that already
    holds `[N/R, ...]` blocks is taken as is), and `state_dict()` returns the `[N, ...]` tensors again by all-gathering
    the blocks, which makes it a COLLECTIVE call: every rank of the group must make it.  Set
    `full_checkpoints = False` to save and load the local blocks only.

    Limits of the peer transport (the default): its buffers hold one step at a time, so a second forward pass before
    the previous one's backward pass raises; and the buffers are (re)allocated collectively, so the call that first
    needs them, or needs larger ones, must be reached by every rank (same token count per rank, or `reserve()` with
    the largest count up front).  Device-side problems (status 301: a peer did not reach a hand-shake in time,
    302: the routing does not fit the buffers, raise `capacity_factor`) are reported as a RuntimeError by the NEXT
    forward pass without synchronising the host; `MOMOE_B200_CHECK=1` reports them at the end of the same pass."""

    def __init__(self, embedding_dim, intermediate_dim, num_experts, num_chosen_experts, num_shared_experts,
                 save_percent=0, bias_update_rate=1e-4, Wg_DN=None, Wl1_ND2H=None, Wl2_NHD=None, *, group=None,
                 transport="peer", capacity_factor=2.0):
        super().__init__()
        assert save_percent >= 0 and save_percent <= 100, \
            "save_percent must be between 0 and 100 inclusive, got {}".format(save_percent)
        self.group = group if group is not None else dist.group.WORLD
        R = dist.get_world_size(self.group)
        assert num_experts % R == 0, "num_experts must be divisible by the number of ranks"
        self.D, self.H, self.N, self.K, self.Ks = (embedding_dim, intermediate_dim, num_experts, num_chosen_experts,
                                                   num_shared_experts)
        self.save_percent = save_percent
        self.bias_update_rate = bias_update_rate
        assert transport in ("peer", "nccl")
        self.transport = transport
        self.capacity_factor = capacity_factor
        self.full_checkpoints = True
        # peer transport, forward pass: 1 = dispatch, GEMMs and combine in sequence; 2 = the local experts in two halves
        # whose transfers overlap the other half's GEMMs (same results bit for bit); None = 2 for large passes
        self.forward_chunks = None
        if os.environ.get("MOMOE_B200_EP_FORWARD_CHUNKS", "") in ("1", "2"):
            self.forward_chunks = int(os.environ["MOMOE_B200_EP_FORWARD_CHUNKS"])
        self._bufs = None
        Nl = num_experts // R
        self.router = TopKRouter(embedding_dim, num_experts, num_chosen_experts, num_shared_experts, Wg_DN=Wg_DN)
        dev = self.router.Wg_DN.device
        if Wl1_ND2H is None:
            Wl1_ND2H = torch.randn((Nl, self.D, 2 * self.H), device=dev, dtype=torch.bfloat16) / self.D
        if Wl2_NHD is None:
            Wl2_NHD = torch.randn((Nl, self.H, self.D), device=dev, dtype=torch.bfloat16) / self.D
        assert Wl1_ND2H.shape[0] == Nl and Wl2_NHD.shape[0] == Nl, "pass this rank's block of N/R experts"
        self.momoe = _ExpertBlock(Wl1_ND2H, Wl2_NHD)
        self.biases_N = nn.Parameter(
            torch.cat([torch.zeros(self.N - self.Ks, device=dev, dtype=torch.float32),
                       torch.full((self.Ks,), float("-inf"), device=dev, dtype=torch.float32)], dim=-1),
            requires_grad=False)
        self._register_load_state_dict_pre_hook(self._shard_checkpoint)
        self._register_state_dict_hook(ExpertParallelMoE._gather_checkpoint)

    # this rank's expert block under the names the single-GPU layer's users know
    @property
    def Wl1_ND2H(self):
        return self.momoe.Wl1_ND2H

    @property
    def Wl2_NHD(self):
        return self.momoe.Wl2_NHD

    def forward(self, x_BSD):
        B, S, _ = x_BSD.shape
        ops.status_poll(self.momoe.Wl1_ND2H.device)    # raises if an earlier pass left a device-side error code
        if self.transport == "peer":
            # compact routing end to end: ids and weights [M,K]; the weights carry the gradient back to the router
            topk_idx, topk_w = CompactRouterFunction.apply(x_BSD, self.router.Wg_DN, self.biases_N, self.N, self.K,
                                                           self.Ks)
            bufs = self._peer_buffers(B * S)
            bufs.forward_chunks = self.forward_chunks
            y_BSD, sizes_N = PeerExpertParallelFunction.apply(x_BSD, self.momoe.Wl1_ND2H, self.momoe.Wl2_NHD,
                                                              topk_idx, topk_w, self.K, self.save_percent, bufs)
        else:
            x_BSD, mask_NM, s_NM = self.router(x_BSD, self.biases_N)
            topk_idx, topk_w = mask_NM._momoe_topk[:2]
            y_BSD, sizes_N = ExpertParallelFunction.apply(x_BSD, self.momoe.Wl1_ND2H, self.momoe.Wl2_NHD, mask_NM,
                                                          s_NM, topk_idx, topk_w, self.K, self.save_percent,
                                                          self.group)
        R = dist.get_world_size(self.group)
        c_avg = B * S * R * (self.K - self.Ks) / (self.N - self.Ks)
        with torch.no_grad():
            ops.bias_update_(self.biases_N.data, sizes_N, self.Ks, c_avg, self.bias_update_rate)
        return y_BSD

    # ---- checkpoints in the single-GPU layout (keys router.Wg_DN, momoe.Wl1_ND2H, momoe.Wl2_NHD, biases_N)
    def _block(self, full):
        R, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        Nl = self.N // R
        return full[rank * Nl:(rank + 1) * Nl]

    def _shard_checkpoint(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        """load_state_dict pre-hook: an `[N, ...]` expert tensor of a single-GPU checkpoint is cut down to this rank's
        block (the dict handed to the hook is load_state_dict's own copy)."""
        for name in ("momoe.Wl1_ND2H", "momoe.Wl2_NHD"):
            key = prefix + name
            t = state_dict.get(key)
            if t is not None and t.dim() == 3 and t.shape[0] == self.N and self.N != self.momoe.Wl1_ND2H.shape[0]:
                state_dict[key] = self._block(t)

    @staticmethod
    def _gather_checkpoint(module, state_dict, prefix, local_metadata):
        """state_dict hook: the expert blocks are all-gathered into the single-GPU `[N, ...]` tensors (collective)."""
        if not module.full_checkpoints or dist.get_world_size(module.group) == 1:
            return
        for name in ("momoe.Wl1_ND2H", "momoe.Wl2_NHD"):
            key = prefix + name
            if key in state_dict:
                state_dict[key] = module._all_gather_blocks(state_dict[key])

    def _all_gather_blocks(self, w):
        R = dist.get_world_size(self.group)
        w = w.detach().contiguous()
        out = torch.empty((R,) + tuple(w.shape), dtype=w.dtype, device=w.device)
        # raw bytes: every backend moves uint8
        dist.all_gather_into_tensor(out.view(torch.uint8).reshape(-1), w.view(torch.uint8).reshape(-1),
                                    group=self.group)
        return out.reshape((R * w.shape[0],) + tuple(w.shape[1:]))

    def load_full_state_dict(self, state):
        """Load a checkpoint of the single-GPU `MoE` layer: every rank keeps its own block of experts.  Same as
        `load_state_dict(state)`; kept for callers of the explicit name."""
        return self.load_state_dict(state)

    def full_state_dict(self):
        """The layer's parameters in the single-GPU layout, on every rank (expert blocks are all-gathered; collective).
        Same as `state_dict()` with `full_checkpoints` set."""
        keep, self.full_checkpoints = self.full_checkpoints, True
        try:
            return {k: v.detach().clone() for k, v in self.state_dict().items()}
        finally:
            self.full_checkpoints = keep

    # ---- peer buffers
    def _rows_for(self, M):
        R = dist.get_world_size(self.group)
        Nl = self.N // R
        # routed experts: capacity_factor x the balanced share; shared experts receive every token of every rank
        want = int(M * (self.K - self.Ks) * self.capacity_factor) + R * M * self.Ks + Nl * 128
        return (want + 127) // 128 * 128

    def reserve(self, max_tokens_per_rank):
        """Allocate the peer buffers for up to `max_tokens_per_rank` tokens on every rank.  COLLECTIVE: every rank of
        the group must call it, with the same value.  Call it up front when ranks will see different token counts."""
        self._bufs = PeerBuffers(self.group, self.momoe.Wl1_ND2H.device, self.N, self.D,
                                 self._rows_for(max_tokens_per_rank))
        self._bufs.max_tokens = max_tokens_per_rank
        return self._bufs

    def _peer_buffers(self, M):
        """Symmetric buffers sized for `capacity_factor` times the average number of rows a rank receives (plus one
        partial tile per local expert).  They are allocated collectively on first use and whenever a rank brings more
        tokens than they were sized for; that call agrees on the largest token count of the group first (one small
        all-reduce and a host read, on that call only), so every rank must reach it."""
        if self._bufs is None or M > self._bufs.max_tokens:
            m = torch.tensor([M], dtype=torch.int64, device=self.momoe.Wl1_ND2H.device)
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=self.group)
            self.reserve(int(m.item()))
        return self._bufs
