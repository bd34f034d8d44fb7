"""GPU parity of the drop-in modules (MoMoE, TopKRouter, MoE) against the golden fixtures produced by the
reference's own kernels and against the CPU oracle.

Tolerances (from the task statement): routing bit-exact; outputs max relative error <= 2e-2 (relative to the
largest reference magnitude); gradients cosine similarity >= 0.999."""
import numpy as np
import pytest
import torch

from helpers import cos, golden_names, load_golden, max_rel
from oracle import momoe_oracle as orc

pytestmark = pytest.mark.gpu

Y_TOL = 2e-2
G_COS = 0.999


@pytest.fixture(scope="module")
def momoe():
    import __graft_entry__
    __graft_entry__.build()
    import momoe
    return momoe


def _check_status():
    from momoe import ops
    torch.cuda.synchronize()
    ops.check_status()


@pytest.mark.parametrize("name", golden_names())
def test_full_layer_against_reference_fixture(momoe, name):
    """TopKRouter -> MoMoE -> bias update, composed as the reference wrapper does, sum-of-squares loss."""
    g = load_golden(name)
    dev = "cuda"
    router = momoe.TopKRouter(g["D"], g["N"], g["K"], g["Ks"], Wg_DN=g["Wg"].to(dev))
    layer = momoe.MoMoE(g["D"], g["H"], g["N"], g["K"], save_percent=g["sp"], Wl1_ND2H=g["W1"].to(dev),
                        Wl2_NHD=g["W2"].to(dev))
    x = g["x"].to(dev).requires_grad_(True)
    xo, mask_NM, s_NM = router(x, g["biases"].to(dev))
    y, sizes = layer(xo, mask_NM, s_NM)
    (y.float() ** 2).sum().backward()
    _check_status()
    # routing: bit-exact
    assert mask_NM.dtype == torch.int32 and tuple(mask_NM.shape) == (g["N"], g["B"] * g["S"])
    assert torch.equal(mask_NM.cpu(), g["mask_NM"])
    assert sizes.dtype == torch.int64 and torch.equal(sizes.cpu(), g["sizes"])
    assert tuple(s_NM.shape) == tuple(g["s_NM"].shape) and s_NM.stride() == (1, g["N"])
    torch.testing.assert_close(s_NM.cpu(), g["s_NM"], rtol=1e-5, atol=1e-8)
    # output and gradients
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == (g["B"], g["S"], g["D"])
    assert max_rel(y.cpu(), g["y"]) <= Y_TOL
    assert cos(y.cpu(), g["y"]) >= 0.9999
    for key, got in (("G_x", x.grad), ("G_W1", layer.Wl1_ND2H.grad), ("G_W2", layer.Wl2_NHD.grad),
                     ("G_Wg", router.Wg_DN.grad)):
        assert got is not None, key
        assert cos(got.cpu(), g[key]) >= G_COS, "%s cos %g" % (key, cos(got.cpu(), g[key]))
        assert max_rel(got.cpu(), g[key]) <= 5e-2, key


@pytest.mark.parametrize("name", golden_names())
def test_experts_with_external_router(momoe, name):
    """MoMoE alone, fed a dense mask_NM / s_NM as an external router would: G_s is dense and zero where unselected."""
    g = load_golden(name)
    dev = "cuda"
    M = g["B"] * g["S"]
    layer = momoe.MoMoE(g["D"], g["H"], g["N"], g["K"], save_percent=g["sp"], Wl1_ND2H=g["W1"].to(dev),
                        Wl2_NHD=g["W2"].to(dev))
    x = g["x"].bfloat16().to(dev).requires_grad_(True)
    s = g["s_NM"].to(dev).clone().requires_grad_(True)
    y, sizes = layer(x, g["mask_NM"].to(dev), s)
    (y.float() ** 2).sum().backward()
    _check_status()
    assert torch.equal(sizes.cpu(), g["sizes"])
    assert max_rel(y.cpu(), g["y"]) <= Y_TOL
    assert tuple(s.grad.shape) == (g["N"], M) and s.grad.dtype == torch.float32
    assert float(s.grad.cpu()[g["mask_NM"] == 0].abs().max()) == 0.0
    assert cos(s.grad.cpu(), g["G_s_NM"]) >= G_COS
    assert cos(x.grad.cpu().reshape(M, -1), g["G_x_experts"].reshape(M, -1)) >= G_COS


LAYER_CASES = [
    # B, S, D, H, N, K, Ks, save_percent, bias_std
    (2, 64, 256, 128, 8, 2, 0, 0, 0.0),
    (2, 512, 512, 256, 16, 4, 1, 37, 0.02),
    (4, 1920, 2176, 1152, 64, 6, 0, 50, 0.0),     # chart shape with D, H not multiples of 128/256
    (1, 333, 192, 136, 12, 5, 2, 100, 0.05),      # ragged everything
    (1, 1, 128, 64, 128, 8, 0, 0, 0.0),           # a single token: 120 experts without tokens
]


@pytest.mark.parametrize("fused", [True, False], ids=["fused", "composed"])
@pytest.mark.parametrize("B,S,D,H,N,K,Ks,sp,bias_std", LAYER_CASES)
def test_moe_wrapper_against_oracle(momoe, B, S, D, H, N, K, Ks, sp, bias_std, fused):
    gen = torch.Generator().manual_seed(B * S + D)
    x = torch.randn(B, S, D, generator=gen)
    W1 = (torch.randn(N, D, 2 * H, generator=gen) * 0.02).bfloat16()
    W2 = (torch.randn(N, H, D, generator=gen) * 0.02).bfloat16()
    Wg = (torch.randn(D, N, generator=gen) * 0.02).bfloat16()
    dev = "cuda"
    moe = momoe.MoE(D, H, N, K, Ks, save_percent=sp, bias_update_rate=1e-3, Wg_DN=Wg.to(dev), Wl1_ND2H=W1.to(dev),
                    Wl2_NHD=W2.to(dev))
    assert sorted(moe.state_dict()) == ["biases_N", "momoe.Wl1_ND2H", "momoe.Wl2_NHD", "router.Wg_DN"]
    moe.fused = fused
    with torch.no_grad():
        moe.biases_N[:N - Ks] = (torch.randn(N - Ks, generator=gen) * bias_std).to(dev)
    biases0 = moe.biases_N.detach().cpu().clone()
    xg = x.to(dev).requires_grad_(True)
    y = moe(xg)
    (y.float() ** 2).sum().backward()
    _check_status()
    # The gate GEMM is a library call on both sides and may round a logit differently; the oracle always routes on
    # the logits the device produced, so every case is checked whatever the rounding.
    logits_dev = (xg.detach().reshape(B * S, D).bfloat16() @ Wg.to(dev)).cpu()
    o = orc.moe_forward_backward(x, Wg, W1, W2, biases0, K, Ks, save_percent=sp, logits=logits_dev)
    sizes = torch.as_tensor(o["sizes"])
    exp_b = orc.bias_update(biases0, sizes, B * S, K, Ks, 1e-3)
    assert torch.equal(moe.biases_N.detach().cpu(), exp_b)
    assert max_rel(y.cpu(), o["y"]) <= Y_TOL
    for key, got in (("G_x", xg.grad), ("G_W1", moe.momoe.Wl1_ND2H.grad), ("G_W2", moe.momoe.Wl2_NHD.grad),
                     ("G_Wg", moe.router.Wg_DN.grad)):
        assert cos(got.cpu(), o[key]) >= G_COS, "%s cos %g" % (key, cos(got.cpu(), o[key]))
    # experts without tokens: exact zero weight gradients
    for e in np.nonzero(o["sizes"] == 0)[0]:
        assert float(moe.momoe.Wl1_ND2H.grad[e].float().abs().sum()) == 0.0
        assert float(moe.momoe.Wl2_NHD.grad[e].float().abs().sum()) == 0.0


@pytest.mark.parametrize("B,S,D,H,N,K,Ks,sp", [(2, 512, 512, 256, 16, 4, 1, 37), (1, 333, 192, 136, 12, 5, 2, 100),
                                               (4, 1024, 1024, 512, 32, 4, 0, 0)])
def test_fused_wrapper_equals_router_then_experts(momoe, B, S, D, H, N, K, Ks, sp):
    """The single-node `MoE` path (compact routing end to end) against the literal TopKRouter -> MoMoE composition:
    same output and expert gradients bit for bit; the gate gradient differs only by fp32 summation order."""
    gen = torch.Generator().manual_seed(7 * S + N)
    dev = "cuda"
    x = torch.randn(B, S, D, generator=gen).to(dev)
    W1 = (torch.randn(N, D, 2 * H, generator=gen) * 0.02).bfloat16().to(dev)
    W2 = (torch.randn(N, H, D, generator=gen) * 0.02).bfloat16().to(dev)
    Wg = (torch.randn(D, N, generator=gen) * 0.02).bfloat16().to(dev)
    g = torch.randn(B, S, D, generator=gen).bfloat16().to(dev)
    out = {}
    for fused in (True, False):
        moe = momoe.MoE(D, H, N, K, Ks, save_percent=sp, Wg_DN=Wg, Wl1_ND2H=W1, Wl2_NHD=W2)
        moe.fused = fused
        xg = x.clone().requires_grad_(True)
        y = moe(xg)
        y.backward(g)
        _check_status()
        out[fused] = (y.detach(), moe.momoe.Wl1_ND2H.grad, moe.momoe.Wl2_NHD.grad, xg.grad, moe.router.Wg_DN.grad,
                      moe.biases_N.detach().clone())
    a, b = out[True], out[False]
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
    assert torch.equal(a[5], b[5])
    assert cos(a[4].cpu(), b[4].cpu()) >= 0.99999 and max_rel(a[4].cpu(), b[4].cpu()) <= 1e-2
    assert cos(a[3].cpu(), b[3].cpu()) >= 0.99999


def test_experts_honour_the_routing_tensors_they_are_given(momoe):
    """`MoMoE` must read the `mask_NM` / `s_NM` it is called with (the reference reads s_NM in its down projection,
    momoe/momoe.py:235-237, and the mask in find_used_experts, :821-842), not what the router attached to them:
    doubled weights double the output exactly, a mask edited in place after routing is honoured, and the compact
    short-cut is only taken for the router's own, unmodified tensors."""
    from momoe.momoe import compact_routing_of
    B, S, D, H, N, K, Ks = 1, 300, 256, 128, 8, 2, 0
    dev = "cuda"
    gen = torch.Generator().manual_seed(11)
    W1 = (torch.randn(N, D, 2 * H, generator=gen) * 0.05).bfloat16().to(dev)
    W2 = (torch.randn(N, H, D, generator=gen) * 0.05).bfloat16().to(dev)
    Wg = (torch.randn(D, N, generator=gen) * 0.05).bfloat16().to(dev)
    x = torch.randn(B, S, D, generator=gen).bfloat16().to(dev)
    router = momoe.TopKRouter(D, N, K, Ks, Wg_DN=Wg)
    layer = momoe.MoMoE(D, H, N, K, save_percent=0, Wl1_ND2H=W1, Wl2_NHD=W2)
    biases = torch.zeros(N, device=dev)
    with torch.no_grad():
        _, mask_NM, s_NM = router(x, biases)
        assert compact_routing_of(mask_NM, s_NM) is not None
        y1, sizes1 = layer(x, mask_NM, s_NM)
        s2 = 2.0 * s_NM
        assert compact_routing_of(mask_NM, s2) is None
        y2, _ = layer(x, mask_NM, s2)
        assert torch.equal(y2.float(), 2.0 * y1.float())      # a power of two commutes with every rounding
        # move token 0 from its first expert to an expert it did not select, as a capacity-dropping caller might
        sel = torch.nonzero(mask_NM[:, 0]).flatten()
        free = [e for e in range(N) if e not in sel.tolist()][0]
        mask3 = mask_NM.clone()
        s3 = s_NM.clone()
        mask3[sel[0], 0], mask3[free, 0] = 0, 1
        s3[free, 0], s3[sel[0], 0] = s3[sel[0], 0].item(), 0.0
        y3, sizes3 = layer(x, mask3, s3)
        assert int(sizes3[free]) == int(sizes1[free]) + 1 and int(sizes3[sel[0]]) == int(sizes1[sel[0]]) - 1
        assert torch.equal(y3[0, 1:], y1[0, 1:]) and not torch.equal(y3[0, 0], y1[0, 0])
        # the same edit done IN PLACE on the router's own tensors must be seen as well
        mask_NM[sel[0], 0], mask_NM[free, 0] = 0, 1
        assert compact_routing_of(mask_NM, s_NM) is None
        y4, _ = layer(x, mask_NM, s3)
        assert torch.equal(y4, y3)
    _check_status()


def test_forward_replays_as_a_cuda_graph(momoe):
    """No host synchronisation and no host-side dependence on the routing: a captured forward pass, replayed on new
    inputs of the same shape, gives what the eager call gives on them (bias update switched off so that both see the
    same biases)."""
    B, S, D, H, N, K, Ks = 1, 96, 256, 128, 16, 4, 1
    dev = "cuda"
    moe = momoe.MoE(D, H, N, K, Ks, save_percent=0, bias_update_rate=0.0)
    gen = torch.Generator(device=dev).manual_seed(2)
    x_static = torch.randn(B, S, D, generator=gen, device=dev).bfloat16()
    with torch.no_grad():
        moe(x_static)                                  # first call: every lazy initialisation happens here
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y_static = moe(x_static)
        for seed in (3, 4):
            x_new = torch.randn(B, S, D, generator=torch.Generator(device=dev).manual_seed(seed), device=dev).bfloat16()
            x_static.copy_(x_new)
            graph.replay()
            torch.cuda.synchronize()
            y_eager = moe(x_new)
            assert torch.equal(y_static, y_eager)
    _check_status()


def test_forward_is_deterministic_and_training_reduces_loss(momoe):
    """Mirror of the reference's only test (momoe/test.py): AdamW on MSE-to-input must go down; plus
    run-to-run bitwise determinism of the forward pass (no atomics anywhere in it)."""
    torch.manual_seed(0)
    B, S, D, H, N, K, Ks = 2, 256, 256, 128, 16, 4, 1
    x = torch.randn(B, S, D, device="cuda", dtype=torch.bfloat16)
    moe = momoe.MoE(D, H, N, K, Ks, save_percent=0, bias_update_rate=1e-4)
    with torch.no_grad():
        y1 = moe(x).clone()
        moe.biases_N[:N - Ks] = 0
        y2 = moe(x).clone()
    assert torch.equal(y1, y2)
    opt = torch.optim.AdamW(moe.parameters(), lr=1e-3)
    losses = []
    for _ in range(30):
        y = moe(x)
        loss = torch.mean(torch.square(y.float() - x.float()))
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss))
    _check_status()
    assert losses[-1] < losses[0] * 0.9, losses


def test_memory_held_for_backward_follows_save_percent(momoe):
    """What the layer keeps alive between forward and backward: the bf16 input, the routing tables and, for the saved
    share of the rows only, the pre-activations a and b (2 * rows * H * 2 bytes).  Nothing else (no [K,M,D] slab, no
    y_pre): the reference's memory chart property."""
    B, S, D, H, N, K = 4, 2048, 1024, 512, 32, 4
    M, Msum = B * S, B * S * K
    g = torch.Generator().manual_seed(0)
    W1 = (torch.randn(N, D, 2 * H, generator=g) * 0.02).bfloat16().cuda()
    W2 = (torch.randn(N, H, D, generator=g) * 0.02).bfloat16().cuda()
    Wg = (torch.randn(D, N, generator=g) * 0.02).bfloat16().cuda()
    x = torch.randn(B, S, D, generator=g).bfloat16().cuda().requires_grad_(True)
    held = {}
    for sp in (0, 50, 100):
        moe = momoe.MoE(D, H, N, K, 0, save_percent=sp, Wg_DN=Wg, Wl1_ND2H=W1, Wl2_NHD=W2)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        before = torch.cuda.memory_allocated()
        y = moe(x)
        torch.cuda.synchronize()
        held[sp] = torch.cuda.memory_allocated() - before - y.numel() * 2
        y.sum().backward()
        del y, moe
    ab_all = 2 * Msum * H * 2
    assert held[0] < 0.35 * ab_all                      # tables + weights cast + router state only
    assert 0.4 * ab_all < held[50] - held[0] < 0.75 * ab_all
    assert 0.9 * ab_all < held[100] - held[0] < 1.35 * ab_all


def test_peer_handshake_gives_up_with_a_status_code(momoe):
    """A wait on a peer that never arrives must run out, record status 301 and return, leaving the context usable
    (failure detection without faulting a GPU: the flag simply is never set).  One GPU plays rank 0 of a 2-rank group
    whose "peer" flag array is a second local buffer that nothing signals; the wait limit is shortened to ~20 ms."""
    import ctypes as C
    from momoe import _lib, ops
    L = _lib.lib
    dev = torch.device("cuda")
    mine = torch.zeros(8, dtype=torch.int32, device=dev)
    peer = torch.zeros(8, dtype=torch.int32, device=dev)
    flags = (C.c_void_p * 2)(C.c_void_p(mine.data_ptr()), C.c_void_p(peer.data_ptr()))
    status = ops.status_word(dev)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    before = L.momoe_ep_set_wait_limit(30_000_000)          # cycles: 15-25 ms at the SM clocks seen here
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        _lib.check(L.momoe_ep_barrier(flags, 2, 0, 1, _lib.ptr(status), _lib.stream_ptr()), "barrier")
        t1.record()
        torch.cuda.synchronize()
        assert 1.0 < t0.elapsed_time(t1) < 500.0             # it waited, and it gave up
        assert peer.tolist()[0] == 1 and mine.tolist()[1] == 0      # our epoch reached the "peer"; nothing came back
        with pytest.raises(RuntimeError, match="301"):
            ops.check_status(dev)
        ops.check_status(dev)                                 # cleared
        # the same hand-shake completes at once when the peer's flag is there
        mine[1] = 2
        _lib.check(L.momoe_ep_barrier(flags, 2, 0, 2, _lib.ptr(status), _lib.stream_ptr()), "barrier")
        torch.cuda.synchronize()
        ops.check_status(dev)
        # and the device still computes
        assert float((torch.ones(1024, device=dev) * 2).sum()) == 2048.0
    finally:
        assert L.momoe_ep_set_wait_limit(before) == 30_000_000


def test_device_error_is_reported_by_the_next_forward_without_a_sync(momoe):
    """The asynchronous status report: a device-side error code left by one pass (here: a mask with a token that lacks
    an expert) raises at a later forward call of the layer, with no `check_status` call by the user."""
    from momoe import ops
    from helpers import dense_from_topk, make_routing
    M, N, K, D, H = 64, 8, 2, 64, 32
    dev = "cuda"
    torch.cuda.synchronize()
    ops.check_status(dev)
    topk_idx, topk_w = make_routing(M, N, K, seed=1)
    mask_NM, s_NM = dense_from_topk(topk_idx, topk_w, N)
    good_mask = mask_NM.clone()
    mask_NM[:, 5] = 0                                         # token 5 has no expert
    layer = momoe.MoMoE(D, H, N, K)
    x = torch.randn(1, M, D, device=dev).bfloat16()
    with torch.no_grad():
        layer(x, mask_NM, s_NM)                               # records 201 on the device; nothing raises here
        torch.cuda.synchronize()                              # (only so that the test is deterministic)
        with pytest.raises(RuntimeError, match="201"):
            for _ in range(3):                                # the report is picked up by one of the next calls
                layer(x, good_mask, s_NM)
                torch.cuda.synchronize()
        layer(x, good_mask, s_NM)                             # and the layer is usable again
    _check_status()
