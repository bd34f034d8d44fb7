"""The expert-parallel transfer kernels on ONE GPU: the device plays a group of one rank whose "peer" buffers are its
own, so every entry point of the peer transport runs where only one GPU is visible (the multi-GPU parity of the whole
layer is tests/test_gpu_ep.py).  Everything here is a row copy, a table or a sum in a fixed order: results must agree
bit for bit."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import make_routing

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import __graft_entry__
    __graft_entry__.build()
    from momoe import _lib, ops
    return _lib, ops


def _one(t):
    return (C.c_void_p * 1)(C.c_void_p(t.data_ptr()))


class _Rank:
    """Buffers and plan of a one-rank group for the routing (topk_idx, topk_w)."""

    def __init__(self, env, M, N, K, D, H, save_percent, seed, split):
        _lib, ops = env
        L, p, st = _lib.lib, _lib.ptr, _lib.stream_ptr
        dev = torch.device("cuda")
        i32 = dict(dtype=torch.int32, device=dev)
        self.env, self.M, self.N, self.K, self.D, self.H, self.split = env, M, N, K, D, H, split
        topk_idx, topk_w = make_routing(M, N, K, seed=seed, skew=1.5)
        self.home = ops.RoutingPlan.from_topk(topk_idx, topk_w, N, D, H, 0.0)
        self.status = self.home.status
        self.cap = self.home.rows_capacity + 256
        self.tile_cap = self.cap // 128
        self.counts = torch.zeros(N, **i32)
        self.flags = torch.zeros(16, **i32)
        _lib.check(L.momoe_ep_publish_counts(p(self.home.sizes), N, _one(self.counts), _one(self.flags), 1, 0, 1,
                                             p(self.status), st()), "publish")
        self.dst_base = torch.empty(N, **i32)
        self.sizes_global = torch.empty(N, dtype=torch.int64, device=dev)
        self.local_count = torch.empty(N, **i32)
        self.pad_off = torch.empty(N + 1, **i32)
        self.tile_expert = torch.full((self.tile_cap,), -1, **i32)
        self.pair_info = torch.full((self.tile_cap,), -1, **i32)
        self.sched = torch.empty(8, **i32)
        self.pair_parts = torch.full((2 * self.tile_cap,), -1, **i32)
        self.sched_parts = torch.empty(16, **i32)
        _lib.check(L.momoe_ep_plan_split(p(self.counts), 1, 0, N, float(save_percent), self.cap, p(self.dst_base),
                                         p(self.sizes_global), p(self.local_count), p(self.pad_off),
                                         p(self.tile_expert), p(self.pair_info), p(self.sched), split,
                                         p(self.pair_parts), p(self.sched_parts), p(self.status), st()), "plan")
        self.row_w = torch.full((self.cap,), float("nan"), device=dev)

    def plan(self, sched, sched_off, pairs, pair_off):
        _lib, _ = self.env
        return _lib.Plan(M=1, N=self.N, K=1, D=self.D, H=self.H, reserved=0, rows_capacity=self.cap,
                         sched=sched.data_ptr() + 4 * sched_off, tile_expert=self.tile_expert.data_ptr(),
                         pad_off=self.pad_off.data_ptr(), row_token=0, row_weight=self.row_w.data_ptr(), pos_MK=0,
                         status=self.status.data_ptr(), pair_info=pairs.data_ptr() + 4 * pair_off)


@pytest.mark.parametrize("M,N,K,D,H,sp,split", [(700, 12, 3, 256, 128, 0, 6), (1500, 8, 2, 384, 136, 50, 3),
                                                 (300, 16, 4, 128, 64, 100, 8),
                                                 # rows that are not a multiple of 32 bytes, K outside {2,4,6,8},
                                                 # an uneven split
                                                 (200, 6, 5, 136, 72, 50, 2)])
def test_split_plan_ranged_dispatch_pull_and_staged_combine(env, M, N, K, D, H, sp, split):
    _lib, ops = env
    L, p, st = _lib.lib, _lib.ptr, _lib.stream_ptr
    dev = torch.device("cuda")
    r = _Rank(env, M, N, K, D, H, sp, seed=M, split=split)
    torch.cuda.synchronize()
    ops.check_status(dev)

    # ---- the plan of a one-rank group is the single-GPU plan, and the two parts partition its pair table
    assert torch.equal(r.sizes_global, r.home.sizes)
    assert torch.equal(r.pad_off, r.home.pad_off)
    n_pairs = int(r.sched[3])
    assert n_pairs == int(r.home.sched[3])
    assert int(r.sched[1]) == int(ops.RoutingPlan.from_topk(r.home.topk_idx, r.home.topk_w, N, D, H, sp).sched[1])
    assert torch.equal(r.pair_info[:n_pairs], r.home.pair_info[:n_pairs])
    sp_ = r.sched_parts.cpu().numpy().reshape(2, 8)
    n0, n1 = int(sp_[0, 3]), int(sp_[1, 3])
    assert n0 + n1 == n_pairs
    assert torch.equal(torch.cat([r.pair_parts[:n0], r.pair_parts[r.tile_cap:r.tile_cap + n1]]), r.pair_info[:n_pairs])
    te = r.tile_expert.cpu().numpy()
    first_tiles0 = (r.pair_parts[:n0].cpu().numpy() >> 1)
    first_tiles1 = (r.pair_parts[r.tile_cap:r.tile_cap + n1].cpu().numpy() >> 1)
    assert np.all(te[first_tiles0] < split) and np.all(te[first_tiles1] >= split)
    assert sp_[0, 1] == sp_[1, 1] == int(r.sched[1]) and sp_[0, 0] == sp_[1, 0] == int(r.sched[0])
    assert sp_[0, 2] + sp_[1, 2] == int(r.sched[2])

    # ---- dispatch: whole block at once against the two ranges; buffers start as NaN so that padding rows must be zeroed
    x = torch.randn(M, D, device=dev).bfloat16()
    nan = float("nan")

    def dispatch(ranges):
        rows = torch.full((r.cap, D), nan, device=dev).bfloat16()
        roww = torch.full((r.cap,), nan, device=dev)
        remote = torch.full((r.home.rows_capacity,), -5, dtype=torch.int32, device=dev)
        for lo, hi in ranges:
            if (lo, hi) == (0, N):
                rc = L.momoe_ep_dispatch_rows(r.home.ref, p(x), D, p(r.dst_base), N, _one(rows), _one(roww), p(remote),
                                              1, 0, p(r.local_count), p(r.pad_off), 0, st())
            else:
                rc = L.momoe_ep_dispatch_rows_range(r.home.ref, p(x), D, p(r.dst_base), N, _one(rows), _one(roww),
                                                    p(remote), 1, 0, p(r.local_count), p(r.pad_off), lo, hi, 148, st())
            _lib.check(rc, "dispatch")
        return rows, roww, remote

    rows_a, roww_a, remote_a = dispatch([(0, N)])
    rows_b, roww_b, remote_b = dispatch([(split, N), (0, split)])
    n_rows = int(r.sched[2])
    assert torch.equal(rows_a[:n_rows].view(torch.int16), rows_b[:n_rows].view(torch.int16))
    assert torch.equal(roww_a[:n_rows], roww_b[:n_rows]) and torch.equal(remote_a, remote_b)
    # one rank: the owner's layout is the home layout, so the dispatch is the plain gather
    ref = ops.gather_rows(r.home, x, D)
    assert torch.equal(rows_a[:n_rows].view(torch.int16), ref[:n_rows].view(torch.int16))
    assert torch.equal(roww_a[:n_rows], r.home.row_weight[:n_rows])

    # ---- the GEMMs of the two parts together do what the GEMMs of the whole block do
    r.row_w.copy_(torch.cat([roww_a, torch.zeros(r.cap - roww_a.numel(), device=dev)])[:r.cap])
    W1 = (torch.randn(N, D, 2 * H, device=dev) * 0.05).bfloat16()
    W2 = (torch.randn(N, H, D, device=dev) * 0.05).bfloat16()
    whole = r.plan(r.sched, 0, r.pair_info, 0)
    parts = [r.plan(r.sched_parts, 0, r.pair_parts, 0), r.plan(r.sched_parts, 8, r.pair_parts, r.tile_cap)]

    def gemms(plans):
        h = torch.zeros((r.cap, H), device=dev).bfloat16()
        y = torch.zeros((r.cap, D), device=dev).bfloat16()
        for pl in plans:
            _lib.check(L.momoe_up_swiglu(C.byref(pl), p(rows_a), p(W1), p(h), None, None, 0, st()), "up")
            _lib.check(L.momoe_down_scale(C.byref(pl), p(h), p(W2), p(y), st()), "down")
        return h, y

    h_a, y_a = gemms([whole])
    h_b, y_b = gemms(parts)
    pos = r.home.pos.long()                      # real rows only: a pair's unused second tile is never written
    assert torch.equal(h_a[pos].view(torch.int16), h_b[pos].view(torch.int16))
    assert torch.equal(y_a[pos].view(torch.int16), y_b[pos].view(torch.int16))

    # ---- combine: straight from the owner against pull + staged combine
    out_a = torch.empty((M, D), device=dev).bfloat16()
    _lib.check(L.momoe_ep_combine_rows(r.home.ref, _one(y_a), p(remote_a), N, D, p(out_a), 1, 0, st()), "combine")
    staged = torch.full((r.home.rows_capacity, D), nan, device=dev).bfloat16()
    _lib.check(L.momoe_ep_pull_rows(r.home.ref, _one(y_a), p(remote_a), N, D, p(staged), 1, 0, 0, split, 148, st()),
               "pull")
    out_b = torch.empty((M, D), device=dev).bfloat16()
    _lib.check(L.momoe_ep_combine_rows_staged(r.home.ref, _one(y_a), p(remote_a), N, D, p(out_b), 1, p(staged), 0, split,
                                              0, st()), "combine staged")
    torch.cuda.synchronize()
    ops.check_status(dev)
    assert torch.isfinite(out_a.float()).all()
    assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))
    assert torch.equal(out_a.view(torch.int16), ops.combine_rows(r.home, y_a, D).view(torch.int16))


def test_range_arguments_are_checked(env):
    _lib, ops = env
    L, p, st = _lib.lib, _lib.ptr, _lib.stream_ptr
    r = _Rank(env, 64, 4, 2, 64, 32, 0, seed=3, split=2)
    x = torch.zeros(64, 64, device="cuda").bfloat16()
    rows = torch.zeros((r.cap, 64), device="cuda").bfloat16()
    remote = torch.zeros(r.home.rows_capacity, dtype=torch.int32, device="cuda")
    for lo, hi in ((-1, 2), (3, 2), (0, 5)):
        assert L.momoe_ep_dispatch_rows_range(r.home.ref, p(x), 64, p(r.dst_base), 4, _one(rows), None, p(remote), 1, 0,
                                              p(r.local_count), p(r.pad_off), lo, hi, 0, st()) == -1
        assert L.momoe_ep_pull_rows(r.home.ref, _one(rows), p(remote), 4, 64, p(rows), 1, 0, lo, hi, 0, st()) == -1
    assert L.momoe_ep_plan_split(p(r.counts), 1, 0, 4, 0.0, r.cap, p(r.dst_base), p(r.sizes_global), p(r.local_count),
                                 p(r.pad_off), p(r.tile_expert), p(r.pair_info), p(r.sched), 9, p(r.pair_parts),
                                 p(r.sched_parts), p(r.status), st()) == -1
    torch.cuda.synchronize()
    ops.check_status("cuda")
