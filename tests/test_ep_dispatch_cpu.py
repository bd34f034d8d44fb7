"""Expert-parallel dispatch metadata with two CPU ranks (gloo): rows reach the rank that owns their expert, arrive in
source-major / expert-major order, and return to the slot they left from."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import momoe_oracle as orc


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _routing(rank, M, N, K):
    g = torch.Generator().manual_seed(100 + rank)
    logits = torch.randn(M, N, generator=g) + (torch.arange(N) % 3 == 0) * 1.5     # skewed
    sel = torch.topk(logits, K, dim=-1).indices
    mask = torch.zeros(M, N, dtype=torch.int32).scatter_(1, sel, 1).T.contiguous()
    sizes, cumsums, idx, which = orc.permutation_from_mask(mask.numpy(), K)
    return torch.from_numpy(sizes), torch.from_numpy(idx), torch.from_numpy(which), mask


def _worker(rank, world, port, M, N, K, D):
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(os.path.dirname(here), "momoe-impl_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from momoe import ep
    sizes, idx, which, mask = _routing(rank, M, N, K)
    Nl = N // world
    sizes_RN = ep.gather_counts(sizes, dist.group.WORLD)
    assert sizes_RN.shape == (world, N) and torch.equal(sizes_RN[rank], sizes)
    meta = ep.DispatchMeta(sizes_RN, idx, which, rank, M, K)
    assert sum(meta.send_splits) == M * K
    assert torch.equal(meta.global_sizes, sizes_RN.sum(0))
    # payload: [global expert, source rank, token, value]
    x = torch.randn(M, D, generator=torch.Generator().manual_seed(7 + rank))
    expert_of_row = torch.from_numpy(np.nonzero(mask.numpy())[0])
    assert torch.equal(meta.send_expert, expert_of_row)
    tag = torch.stack([expert_of_row.float(), torch.full((M * K,), float(rank)), idx.float()], dim=1)
    send = torch.cat([tag, x[idx.long()]], dim=1)
    recv = ep.exchange(send, meta.send_splits, meta.recv_splits, dist.group.WORLD)
    assert recv.shape[0] == meta.n_recv == int(sizes_RN[:, rank * Nl:(rank + 1) * Nl].sum())
    # every received row belongs to one of this rank's experts, and recv_expert names it
    assert torch.equal(recv[:, 0].long() - rank * Nl, meta.recv_expert.long())
    # source-major, then expert-major, then ascending token
    key = recv[:, 1].double() * 1e9 + recv[:, 0].double() * 1e5 + recv[:, 2].double()
    assert torch.all(key[1:] > key[:-1])
    # "expert" e multiplies by (e + 1); send back and combine at home
    y_recv = recv[:, 3:] * (recv[:, 0:1] + 1.0)
    y_back = ep.exchange(y_recv, meta.recv_splits, meta.send_splits, dist.group.WORLD)
    pos = meta.pos_unpadded.view(M, K).long()
    y = y_back[pos].sum(1)
    expect = x * (mask.T.float() @ (torch.arange(N).float() + 1.0))[:, None]
    torch.testing.assert_close(y, expect, rtol=1e-5, atol=1e-5)
    # slot k of token m is its k-th expert in ascending id
    assert torch.equal(expert_of_row[pos], torch.sort(torch.nonzero(mask.T)[:, 1].view(M, K), dim=1).values)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,M,N,K", [(2, 50, 8, 2), (2, 33, 6, 3), (4, 40, 8, 4)])
def test_dispatch_round_trip_gloo(world, M, N, K):
    mp.spawn(_worker, args=(world, _free_port(), M, N, K, 5), nprocs=world, join=True)


def _ckpt_worker(rank, world, port):
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(os.path.dirname(here), "momoe-impl_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from momoe import ep
    D, H, N, K, Ks = 16, 8, 6, 3, 1
    g = torch.Generator().manual_seed(0)     # the same "checkpoint" on every rank
    full = {"router.Wg_DN": torch.randn(D, N, generator=g).bfloat16(),
            "momoe.Wl1_ND2H": torch.randn(N, D, 2 * H, generator=g).bfloat16(),
            "momoe.Wl2_NHD": torch.randn(N, H, D, generator=g).bfloat16(),
            "biases_N": torch.cat([torch.randn(N - Ks, generator=g), torch.full((Ks,), float("-inf"))])}
    Nl = N // world
    moe = ep.ExpertParallelMoE(D, H, N, K, Ks, Wg_DN=torch.zeros(D, N), Wl1_ND2H=torch.zeros(Nl, D, 2 * H),
                               Wl2_NHD=torch.zeros(Nl, H, D), transport="nccl")
    # the sharded layer exposes the single-GPU layer's keys ...
    assert sorted(k for k, _ in moe.named_parameters()) == sorted(full)
    # ... and a plain load_state_dict of a single-GPU checkpoint keeps this rank's expert block (strict: no missing or
    # unexpected keys, no shape errors)
    res = moe.load_state_dict(full)
    assert not res.missing_keys and not res.unexpected_keys
    assert torch.equal(moe.Wl1_ND2H, full["momoe.Wl1_ND2H"][rank * Nl:(rank + 1) * Nl])
    assert torch.equal(moe.Wl2_NHD, full["momoe.Wl2_NHD"][rank * Nl:(rank + 1) * Nl])
    assert torch.equal(moe.router.Wg_DN, full["router.Wg_DN"]) and torch.equal(moe.biases_N, full["biases_N"])
    assert full["momoe.Wl1_ND2H"].shape[0] == N                    # the caller's dict is left as it was
    # state_dict() gives the single-GPU layout back, bit for bit (collective all-gather of the blocks)
    back = moe.state_dict()
    assert sorted(back) == sorted(full)
    for k in full:
        assert torch.equal(back[k], full[k]), k
    # the explicit helpers are the same thing
    moe2 = ep.ExpertParallelMoE(D, H, N, K, Ks, Wg_DN=torch.zeros(D, N), Wl1_ND2H=torch.zeros(Nl, D, 2 * H),
                                Wl2_NHD=torch.zeros(Nl, H, D), transport="nccl")
    moe2.load_full_state_dict(full)
    for k, v in moe2.full_state_dict().items():
        assert torch.equal(v, full[k]), k
    # local-block checkpoints: saved without the gather, loaded as they are
    moe.full_checkpoints = False
    local = moe.state_dict()
    assert tuple(local["momoe.Wl1_ND2H"].shape) == (Nl, D, 2 * H)
    moe2.load_state_dict({k: torch.zeros_like(v) if k.startswith("momoe.") else v for k, v in local.items()})
    assert float(moe2.Wl1_ND2H.float().abs().sum()) == 0.0
    moe2.load_state_dict(local)
    assert torch.equal(moe2.Wl1_ND2H, moe.Wl1_ND2H) and torch.equal(moe2.Wl2_NHD, moe.Wl2_NHD)
    dist.barrier()
    dist.destroy_process_group()


def test_checkpoint_round_trip_in_single_gpu_layout():
    """A checkpoint of the single-GPU layer (the reference's keys: momoe/sample_moe.py:39-57, momoe/momoe.py:947-955)
    loads into the sharded layer with a plain `load_state_dict` and `state_dict()` returns it bit-identical (2 and 3 CPU
    ranks)."""
    mp.spawn(_ckpt_worker, args=(2, _free_port()), nprocs=2, join=True)
    mp.spawn(_ckpt_worker, args=(3, _free_port()), nprocs=3, join=True)


def _failing_worker(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        # this rank dies between steps, before the counts exchange
        os._exit(0)
    t = torch.zeros(4, dtype=torch.int64)
    out = torch.empty(world * 4, dtype=torch.int64)
    try:
        dist.all_gather_into_tensor(out, t)
    except Exception:
        os._exit(0)     # the surviving rank got an error instead of hanging
    os._exit(3)


def test_missing_rank_ends_counts_exchange_with_an_error():
    """A rank that leaves before the counts all-gather must make its peer fail within the group timeout."""
    ctx = mp.spawn(_failing_worker, args=(2, _free_port()), nprocs=2, join=False)
    import time
    deadline = time.time() + 90
    while time.time() < deadline and any(p.exitcode is None for p in ctx.processes):
        time.sleep(0.2)
    codes = [p.exitcode for p in ctx.processes]
    for p in ctx.processes:
        if p.is_alive():
            p.kill()
    assert codes == [0, 0], codes


def _dispatch_visit_order(seg_len, rank, warps_total):
    """Host restatement of the row schedule of ep_dispatch_rows_kernel (csrc/ep.cu): slot j of the grid-stride loop
    -> (destination rank, offset inside that destination's segment of the expert-major rows), or None."""
    world = len(seg_len)
    max_len = max(seg_len)
    rotate = warps_total % world == 0
    visits = []
    for wid in range(warps_total):
        j = wid
        while j < max_len * world:
            off = j // world
            d = j - off * world
            if rotate:
                d = (d + j // warps_total) % world
            d += rank + 1
            if d >= world:
                d -= world
            if off < seg_len[d]:
                visits.append((wid, j // warps_total, d, off))
            j += warps_total
    return visits


@pytest.mark.parametrize("world,warps_total", [(1, 8), (2, 8), (2, 1184), (4, 1184), (8, 9472), (8, 1184), (3, 8), (6, 40)])
def test_dispatch_schedule_visits_every_row_once_and_spreads_destinations(world, warps_total):
    rng = np.random.default_rng(world * 1000 + warps_total)
    seg_len = [int(v) * 128 for v in rng.integers(0, 40, size=world)]
    seg_len[rng.integers(0, world)] = 40 * 128          # at least one long segment
    for rank in range(world):
        visits = _dispatch_visit_order(seg_len, rank, warps_total)
        seen = sorted((d, off) for _, _, d, off in visits)
        want = sorted((d, off) for d in range(world) for off in range(seg_len[d]))
        assert seen == want                              # a bijection onto the rows, whatever the warp count
        if world > 1 and warps_total % world == 0:
            # in one pass of the grid the warps address every destination equally often, the next rank first ...
            first = [d for wid, it, d, off in visits if it == 0]
            if min(seg_len) > warps_total // world:
                counts = np.bincount(first, minlength=world)
                assert counts.min() == counts.max()
            # ... and a warp changes destination from one of its rows to the next
            w0 = [d for wid, it, d, off in visits if wid == 0][:world]
            if min(seg_len) > (world * warps_total) // world:
                assert len(set(w0)) == world


@pytest.mark.parametrize("world,Nl,split", [(2, 4, 2), (8, 16, 8), (4, 3, 1), (8, 2, 1)])
def test_two_expert_ranges_partition_the_rows_of_every_destination(world, Nl, split):
    """ep_dispatch_rows_range / ep_pull_rows (csrc/ep.cu) visit, for destination d and local experts [lo, hi), the run
    [pad_off[d*Nl + lo], pad_off[d*Nl + hi]) of the sender's expert-major rows with the same round-robin schedule.  The
    two halves of a forward pass, (0, split) and (split, Nl), must together visit every row exactly once."""
    rng = np.random.default_rng(world * 100 + Nl)
    padded = rng.integers(0, 6, size=world * Nl) * 128               # padded rows per (global) expert, some empty
    pad_off = np.concatenate([[0], np.cumsum(padded)])
    seen = []
    for lo, hi in ((0, split), (split, Nl)):
        starts = [int(pad_off[d * Nl + lo]) for d in range(world)]
        seg_len = [int(pad_off[d * Nl + hi]) - starts[d] for d in range(world)]
        for _, _, d, off in _dispatch_visit_order(seg_len, rank=1 % world, warps_total=8 * world):
            seen.append(starts[d] + off)
    assert sorted(seen) == list(range(int(pad_off[-1])))


def test_peer_buffers_refuse_a_second_forward_before_the_backward():
    """The peer transport's buffers hold one step at a time (host logic only; no device memory is touched here): a
    forward pass that needs a backward pass blocks the next forward until that backward pass has run or its autograd
    graph has been dropped; passes under no_grad never block."""
    import gc
    import sys
    import weakref
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(os.path.dirname(here), "momoe-impl_b200"))
    from momoe import ep
    bufs = ep.PeerBuffers.__new__(ep.PeerBuffers)      # the bookkeeping without the symmetric allocations
    bufs._step, bufs._pending = 0, 0
    s1 = bufs.begin_step(needs_backward=False)         # inference passes do not hold the buffers
    s2 = bufs.begin_step(needs_backward=True)
    assert (s1, s2) == (1, 2)
    with pytest.raises(RuntimeError, match="backward pass of the previous forward"):
        bufs.begin_step(needs_backward=True)
    with pytest.raises(RuntimeError, match="backward pass of the previous forward"):
        bufs.begin_step(needs_backward=False)          # an evaluation pass in between would overwrite them as well
    bufs.end_step(s1)                                  # a stale step id releases nothing
    with pytest.raises(RuntimeError):
        bufs.begin_step(needs_backward=True)
    bufs.end_step(s2)                                  # the backward pass ran
    s3 = bufs.begin_step(needs_backward=True)
    # an output dropped without a backward pass: the token dies with the graph and releases the buffers
    tok = ep._StepToken()
    weakref.finalize(tok, bufs.end_step, s3)
    del tok
    gc.collect()
    assert bufs.begin_step(needs_backward=True) == s3 + 1
