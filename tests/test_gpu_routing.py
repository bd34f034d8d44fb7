"""GPU parity of the router, the permutation builder and the row movers (all through the C ABI).
Integer outputs are compared bit for bit; fp32 routing weights to 1e-6."""
import numpy as np
import pytest
import torch

from helpers import dense_from_topk, make_routing
from oracle import momoe_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import __graft_entry__
    __graft_entry__.build()
    from momoe import ops
    return ops


ROUTER_CASES = [
    # M, N, K, Ks, bias_std, logit_scale
    (128, 8, 2, 0, 0.0, 1.0),
    (1000, 128, 8, 0, 0.0, 0.05),     # near-uniform bf16 logits: many exact ties at the k-th boundary
    (16384, 128, 8, 0, 0.0, 0.9),
    (4096, 128, 8, 0, 0.5, 1.0),
    (2048, 64, 8, 4, 0.01, 0.3),
    (777, 6, 3, 1, 0.05, 1.0),
    (512, 256, 8, 0, 0.2, 1.0),
    (300, 33, 5, 2, 0.1, 1.0),
    (64, 1024, 8, 0, 0.0, 1.0),
]


@pytest.mark.parametrize("M,N,K,Ks,bias_std,scale", ROUTER_CASES)
def test_route_topk_matches_reference_ops(ops, M, N, K, Ks, bias_std, scale):
    g = torch.Generator().manual_seed(M + N)
    logits = (torch.randn(M, N, generator=g) * scale).bfloat16().cuda()
    biases = torch.cat([torch.randn(N - Ks, generator=g) * bias_std, torch.full((Ks,), float("-inf"))]).cuda()
    topk_idx, topk_w, d = ops.route_topk(logits, biases, K, Ks, dense=True)
    torch.cuda.synchronize()
    # the reference's own sequence of torch calls on the same device (torch.softmax, torch.topk)
    r = orc.router_from_logits(logits, biases, K, Ks, torch_topk=True)
    assert torch.equal(d["mask_NM"], r["mask_NM"]), "selected experts differ from torch.topk on CUDA"
    assert torch.equal(topk_idx, r["topk_idx"])
    # and the documented tie rule (lowest expert id among equal scores) gives the same sets
    r2 = orc.router_from_logits(logits, biases, K, Ks, torch_topk=False)
    assert torch.equal(r2["mask_NM"], r["mask_NM"])
    torch.testing.assert_close(d["s_MN"], r["s_MN"], rtol=1e-6, atol=1e-9)
    torch.testing.assert_close(d["s_postsoft_MN"], r["s_postsoft_MN"], rtol=1e-6, atol=1e-9)
    torch.testing.assert_close(d["Ng_M"], r["Ng_M"], rtol=1e-6, atol=0)
    torch.testing.assert_close(d["Ks_M"], r["Ks_M"], rtol=1e-6, atol=0)
    torch.testing.assert_close(topk_w, torch.gather(r["s_MN"], 1, topk_idx.long()), rtol=1e-6, atol=1e-9)


def test_softmax_probabilities_bit_identical(ops):
    """The warp softmax evaluates exp and the sum in torch's order, so unselected-independent values
    (s_postsoft on the selected entries) are the same bits, which makes biased selection robust."""
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(4096, 128, generator=g).bfloat16().cuda()
    biases = torch.zeros(128).cuda()
    _, _, d = ops.route_topk(logits, biases, 8, 0, dense=True)
    p = torch.softmax(logits, dim=-1, dtype=torch.float32)
    sel = d["mask_NM"].T.bool()
    assert torch.equal(d["s_postsoft_MN"][sel], p[sel])


PERM_CASES = [(128, 8, 2, 0.0), (16384, 128, 8, 0.0), (5000, 64, 6, 2.0), (1, 128, 8, 0.0), (33, 16, 4, 3.0),
              (4096, 256, 8, 1.0), (257, 1024, 8, 0.0)]


@pytest.mark.parametrize("M,N,K,skew", PERM_CASES)
def test_permutation_bit_exact(ops, M, N, K, skew):
    topk_idx, topk_w = make_routing(M, N, K, seed=M * 7 + N, skew=skew)
    plan = ops.RoutingPlan.from_topk(topk_idx, topk_w, N, 64, 64, save_percent=37)
    torch.cuda.synchronize()
    ops.check_status()
    mask_NM, s_NM = dense_from_topk(topk_idx, topk_w, N)
    sizes, cumsums, idx, which = orc.permutation_from_mask(mask_NM.cpu().numpy(), K)
    assert np.array_equal(plan.sizes.cpu().numpy(), sizes)
    assert plan.sizes.dtype == torch.int64
    assert np.array_equal(plan.cumsums.cpu().numpy(), cumsums)
    assert np.array_equal(plan.idx.cpu().numpy(), idx)
    assert np.array_equal(plan.which.cpu().numpy(), which)
    # padded tables
    pad = plan.pad_off.cpu().numpy()
    sched = plan.sched.cpu().numpy()
    exp_pad = np.concatenate([[0], np.cumsum((sizes + 127) // 128 * 128)])
    assert np.array_equal(pad, exp_pad)
    assert sched[0] == exp_pad[-1] // 128 and sched[2] == exp_pad[-1]
    te = plan.tile_expert.cpu().numpy()[:sched[0]]
    assert np.array_equal(te, np.repeat(np.arange(N), (sizes + 127) // 128))
    # pairs: two consecutive tiles of one expert, the last pair of an expert with an odd tile count is single
    ntile = (sizes + 127) // 128
    first = np.concatenate([[0], np.cumsum(ntile)])
    exp_pairs = [int((first[e] + 2 * j) * 2 + (1 if 2 * j + 1 < ntile[e] else 0)) for e in range(N)
                 for j in range((int(ntile[e]) + 1) // 2)]
    assert sched[3] == len(exp_pairs)
    assert plan.pair_info.cpu().numpy()[:sched[3]].tolist() == exp_pairs
    # tiles whose 128-row span (in the unpadded order) ends at or below save_rows
    ends = np.concatenate([cumsums[e] + 128 * (1 + np.arange((sizes[e] + 127) // 128)) for e in range(N)])
    assert sched[1] == int((ends <= plan.save_rows).sum())
    assert np.all(np.diff(ends) > 0)
    rt = plan.row_token.cpu().numpy()[:sched[2]]
    rw = plan.row_weight.cpu().numpy()[:sched[2]]
    pos = plan.pos.cpu().numpy().reshape(M, K)
    tw = topk_w.cpu().numpy()
    ti = topk_idx.cpu().numpy()
    for e in range(N):
        seg = rt[pad[e]:pad[e + 1]]
        assert np.array_equal(seg[:sizes[e]], idx[cumsums[e]:cumsums[e + 1]])
        assert np.all(seg[sizes[e]:] == -1) and np.all(rw[pad[e] + sizes[e]:pad[e + 1]] == 0)
    assert np.array_equal(rt[pos], np.repeat(np.arange(M)[:, None], K, 1))
    assert np.array_equal(rw[pos], tw)
    assert np.array_equal(te[pos // 128], ti)


def test_plan_from_external_mask_with_strides(ops):
    M, N, K = 3000, 40, 5
    topk_idx, topk_w = make_routing(M, N, K, seed=3, skew=1.0)
    mask_NM, s_NM = dense_from_topk(topk_idx, topk_w, N)          # s_NM is a transposed view: strides (1, N)
    assert s_NM.stride() == (1, N)
    plan = ops.RoutingPlan.from_mask(mask_NM, s_NM, K, 64, 64)
    plan2 = ops.RoutingPlan.from_mask(mask_NM.T.contiguous().T, s_NM.contiguous(), K, 64, 64)
    torch.cuda.synchronize()
    ops.check_status()
    for p in (plan, plan2):
        assert torch.equal(p.topk_idx, topk_idx)
        assert torch.equal(p.topk_w, topk_w)
        assert torch.equal(p.idx.long(), torch.nonzero(mask_NM)[:, 1])


def test_mask_without_exactly_k_experts_is_reported(ops):
    M, N, K = 64, 8, 2
    topk_idx, topk_w = make_routing(M, N, K, seed=1)
    mask_NM, s_NM = dense_from_topk(topk_idx, topk_w, N)
    mask_NM[:, 5] = 0
    ops.RoutingPlan.from_mask(mask_NM, s_NM, K, 64, 64)
    with pytest.raises(RuntimeError, match="exactly K"):
        ops.check_status()
    ops.check_status()  # cleared


@pytest.mark.parametrize("M,N,K,D", [(128, 8, 2, 256), (4096, 64, 8, 2048), (1000, 16, 6, 2176), (5, 128, 8, 72)])
def test_gather_and_combine_rows(ops, M, N, K, D):
    topk_idx, topk_w = make_routing(M, N, K, seed=11, skew=1.0)
    plan = ops.RoutingPlan.from_topk(topk_idx, topk_w, N, D, 64)
    x = torch.randn(M, D, generator=torch.Generator().manual_seed(2)).bfloat16().cuda()
    xs = ops.gather_rows(plan, x, D)
    torch.cuda.synchronize()
    rows = int(plan.sched[2])
    rt = plan.row_token[:rows].long()
    expect = torch.where((rt >= 0)[:, None], x[rt.clamp_min(0)], torch.zeros((), dtype=x.dtype, device="cuda"))
    assert torch.equal(xs[:rows], expect)                       # byte-exact move
    # combine: fp32 sum over the token's K rows in ascending k, one rounding to bf16
    ys = torch.randn(plan.rows_capacity, D, generator=torch.Generator().manual_seed(3)).bfloat16().cuda()
    y = ops.combine_rows(plan, ys, D)
    ref = torch.zeros(M, D, device="cuda")
    pos = plan.pos.view(M, K).long()
    for k in range(K):
        ref += ys[pos[:, k]].float()
    assert torch.equal(y, ref.bfloat16())
    # round trip: gathering then combining with K copies gives K*x up to one bf16 rounding
    back = ops.combine_rows(plan, xs, D)
    assert torch.equal(back, (x.float() * K).bfloat16())


@pytest.mark.parametrize("M,n_rows,D", [(64, 200, 256), (4096, 10000, 2048), (7, 3, 72), (1000, 12345, 2176)])
def test_gather_rows_from_a_row_table_only(ops, M, n_rows, D):
    """`momoe_gather_rows` with `plan->pos_MK == NULL`: rows are fetched one by one from `plan->row_token` (the form
    the expert-parallel NCCL transport uses with ad-hoc row tables, including rows marked -1).  Byte-exact against
    `x[row_index]`, through the same helper that transport calls."""
    from momoe import ep
    g = torch.Generator().manual_seed(M + n_rows)
    x = torch.randn(M, D, generator=g).bfloat16().cuda()
    row_index = torch.randint(0, M, (n_rows,), generator=g).to(torch.int32)
    row_index[::7] = -1                                          # padding rows: zeros
    row_index = row_index.cuda()
    got = ep._Rows.gather(x, row_index, n_rows)
    torch.cuda.synchronize()
    ri = row_index.long()
    expect = torch.where((ri >= 0)[:, None], x[ri.clamp_min(0)], torch.zeros((), dtype=x.dtype, device="cuda"))
    assert got.shape == (n_rows, D) and torch.equal(got, expect)
    # and the matching combine with an ad-hoc position table
    K = 3
    Mc = n_rows // K
    pos = torch.randperm(n_rows, generator=g)[:Mc * K].to(torch.int32).cuda()
    y = ep._Rows.combine(got, pos, Mc, K)
    ref = got[pos.long()].float().view(Mc, K, D)
    acc = torch.zeros(Mc, D, device="cuda")
    for k in range(K):
        acc += ref[:, k]
    assert torch.equal(y, acc.bfloat16())
