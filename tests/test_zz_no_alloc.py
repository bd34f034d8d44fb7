"""The allocation-free permutation builder (`momoe_build_permutation_static`) against the regular entry point.

Some hosts of the library cannot allocate device memory at the moment they route tokens (a serving engine whose
pool owns all of HBM, a loop that must not trigger the synchronisation an allocation implies).  For them the
builder's scratch histogram lives in a fixed 1 MiB array inside the library.  This file is collected last on
purpose: should it fail, a run that stops at the first failure has already executed every other test.
"""
import ctypes as C

import pytest
import torch

from helpers import make_routing


@pytest.fixture(scope="module")
def libs():
    import __graft_entry__
    __graft_entry__.build()
    from momoe import _lib
    return _lib


class _Out:
    """Every output buffer of the permutation builder, poisoned so that untouched entries show up."""

    def __init__(self, L, M, N, K, device="cuda"):
        self.rows = int(L.momoe_sorted_rows_capacity(M, K, N))
        tiles = int(L.momoe_tile_capacity(M, K, N))
        i32 = dict(dtype=torch.int32, device=device)
        self.sizes = torch.full((N,), -7, dtype=torch.int64, device=device)
        self.cumsums = torch.full((N + 1,), -7, **i32)
        self.idx = torch.full((M * K,), -7, **i32)
        self.which = torch.full((M * K,), -7, **i32)
        self.pad_off = torch.full((N + 1,), -7, **i32)
        self.tile_expert = torch.full((tiles,), -7, **i32)
        self.pair_info = torch.full((tiles,), -7, **i32)
        self.sched = torch.full((8,), -7, **i32)
        self.row_token = torch.full((self.rows,), -7, **i32)
        self.row_weight = torch.full((self.rows,), -7.0, dtype=torch.float32, device=device)
        self.pos = torch.full((M * K,), -7, **i32)

    def tensors(self, n_tiles=None):
        te = self.tile_expert if n_tiles is None else self.tile_expert[:n_tiles]
        pi = self.pair_info if n_tiles is None else self.pair_info[:int(self.sched[3])]
        return [self.sizes, self.cumsums, self.idx, self.which, self.pad_off, te, pi, self.sched, self.row_token,
                self.row_weight, self.pos]


def _run_both(_lib, M, N, K, seed, save_rows, device="cuda"):
    L, p = _lib.lib, _lib.ptr
    topk_idx, topk_w = make_routing(M, N, K, seed=seed, skew=1.0, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    a, b = _Out(L, M, N, K, device), _Out(L, M, N, K, device)
    nbytes = int(L.momoe_permutation_workspace_bytes(M, N, K))
    ws = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=device)
    st = _lib.stream_ptr()
    rc = L.momoe_build_permutation(p(topk_idx), p(topk_w), M, N, K, save_rows, p(a.sizes), p(a.cumsums), p(a.idx),
                                   p(a.which), p(a.pad_off), p(a.tile_expert), p(a.pair_info), p(a.sched), p(a.row_token),
                                   p(a.row_weight), p(a.pos), a.rows, p(ws), nbytes, p(status), st)
    assert rc == 0
    rc = L.momoe_build_permutation_static(p(topk_idx), p(topk_w), M, N, K, save_rows, p(b.sizes), p(b.cumsums),
                                          p(b.idx), p(b.which), p(b.pad_off), p(b.tile_expert), p(b.pair_info), p(b.sched),
                                          p(b.row_token), p(b.row_weight), p(b.pos), b.rows, p(status), st)
    assert rc == 0
    torch.cuda.synchronize(device)
    assert int(status.item()) == 0
    n_tiles = int(a.sched[0])
    for ta, tb in zip(a.tensors(n_tiles), b.tensors(n_tiles)):
        assert torch.equal(ta, tb)          # integer tables and copied weights: identical bits
    assert int(a.sizes.sum()) == M * K


@pytest.mark.gpu
def test_static_scratch_matches_workspace_version_twice_in_a_row(libs):
    # two different problems back to back: the second call finds the first call's histogram in the shared array
    _run_both(libs, 16384, 128, 8, seed=1, save_rows=50000)
    _run_both(libs, 3000, 40, 5, seed=2, save_rows=0)
    _run_both(libs, 16384, 128, 8, seed=3, save_rows=131072)


@pytest.mark.gpu
def test_static_scratch_small_batch_capacity_edge_and_second_device(libs):
    # a batch small enough for the regular entry point to take its single-launch kernel: the two entry points then run
    # different kernels and must still agree
    assert libs.lib.momoe_permutation_launches(300, 16, 2) == 1
    _run_both(libs, 300, 16, 2, seed=4, save_rows=100)
    # exactly at the capacity of the fixed array: ceil(65536 / 64) * 256 == 262144 ints
    _run_both(libs, 65536, 256, 8, seed=5, save_rows=0)
    _run_both(libs, 300, 16, 2, seed=6, save_rows=0)     # and a small one over the big one's leftovers
    if torch.cuda.device_count() > 1:
        # the array's device address is looked up per device: the same problem on the second GPU
        with torch.cuda.device(1):
            _run_both(libs, 3000, 40, 5, seed=2, save_rows=0, device="cuda:1")
            _run_both(libs, 16384, 128, 8, seed=1, save_rows=50000, device="cuda:1")


def test_static_scratch_rejects_problems_beyond_its_capacity(libs):
    """ceil(M/64) * N must not exceed 262144 ints; the check runs on the host before anything is launched."""
    L = libs.lib
    one = C.c_void_p(16)   # never dereferenced: validation fails first
    M, N, K = 65536 + 64, 256, 8
    rows = int(L.momoe_sorted_rows_capacity(M, K, N))
    args = [one, one, M, N, K, 0] + [one] * 11 + [rows, one, None]
    assert L.momoe_build_permutation_static(*args) == -4
    assert L.momoe_build_permutation_static(None, *args[1:]) == -1
