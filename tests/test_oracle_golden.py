"""The CPU oracle against fixtures produced by the reference's own kernels (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from helpers import cos, golden_names, load_golden, max_rel
from oracle import momoe_oracle as orc


@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_reference_fixture(name):
    g = load_golden(name)
    o = orc.moe_forward_backward(g["x"], g["Wg"], g["W1"], g["W2"], g["biases"], g["K"], g["Ks"],
                                 save_percent=g["sp"], block_rows=g["block_rows"])
    # integers: bit-exact
    assert torch.equal(o["mask_NM"], g["mask_NM"])
    assert np.array_equal(o["sizes"], g["sizes"].numpy())
    assert np.array_equal(o["cumsums"], g["cumsums"].numpy())
    assert np.array_equal(o["idx"], g["idx"].numpy())
    assert np.array_equal(o["which"], g["which"].numpy())
    # routing weights and bias update: fp32, same formulas
    torch.testing.assert_close(o["s_MN"].T, g["s_NM"], rtol=1e-6, atol=1e-7)
    torch.testing.assert_close(o["new_biases"], g["new_biases"], rtol=0, atol=0)
    # outputs and gradients: the fixtures accumulate tile by tile, the oracle in one matmul, so an
    # occasional bf16 rounding flips; everything else is identical
    assert max_rel(o["y"], g["y"]) < 4e-3
    assert cos(o["y"], g["y"]) > 0.99999
    for k in ("G_W1", "G_W2", "G_Wg", "G_x"):
        assert cos(o[k], g[k]) > 0.9999, k
        assert max_rel(o[k], g[k]) < 1e-2, k


@pytest.mark.parametrize("name", golden_names())
def test_oracle_expert_gradients(name):
    """Experts alone with leaf x and s: G_s (dense, zero where unselected) and the experts' own G_x."""
    g = load_golden(name)
    M = g["B"] * g["S"]
    x = g["x"].reshape(M, g["D"]).bfloat16()
    sizes, cumsums, idx, which = orc.permutation_from_mask(g["mask_NM"].numpy(), g["K"])
    y, fwd = orc.experts_forward(x, g["W1"], g["W2"], g["s_NM"], idx, cumsums, which, g["K"])
    G_x, G_W1, G_W2, G_s = orc.experts_backward(2.0 * y.float(), x, g["W1"], g["W2"], g["s_NM"], idx, cumsums,
                                                which, g["K"], g["sp"], fwd, g["block_rows"])
    assert float(G_s[g["mask_NM"] == 0].abs().max()) == 0.0
    assert cos(G_s, g["G_s_NM"]) > 0.9999
    assert max_rel(G_s, g["G_s_NM"]) < 1e-2
    gx_ref = g["G_x_experts"].reshape(M, g["D"])
    assert cos(G_x, gx_ref) > 0.9999
    assert max_rel(G_x, gx_ref) < 1e-2


def test_topk_tie_rule():
    s = torch.tensor([[0.5, 0.25, 0.5, 0.5, 0.1]])
    assert orc.topk_lowest_index_first(s, 2).tolist() == [[0, 2]]
    assert orc.topk_lowest_index_first(s, 4).tolist() == [[0, 1, 2, 3]]


def test_permutation_matches_nonzero():
    rng = np.random.default_rng(0)
    N, M, K = 7, 50, 3
    mask = np.zeros((N, M), dtype=np.int32)
    for m in range(M):
        mask[rng.choice(N, K, replace=False), m] = 1
    sizes, cumsums, idx, which = orc.permutation_from_mask(mask, K)
    assert np.array_equal(idx, np.nonzero(mask)[1])
    assert cumsums[-1] == M * K and sizes.sum() == M * K
    for m in range(M):
        assert sorted(which[idx == m].tolist()) == list(range(K))
