"""Parity at the benchmark's full sizes, through checks whose cost does not grow with the problem.

* routing: the device's selection against the reference's own torch calls on the same logits (bit-exact), and the
  integer invariants of the permutation;
* a random subset of tokens: a token's output, input gradient and routing-weight gradient depend only on its own row
  and on the weights, so the CPU oracle recomputes exactly those tokens (tolerances of the task statement: output
  max-rel <= 2e-2, gradient cosine >= 0.999);
* three experts: their weight gradients against an fp32 torch restatement of the reference math on the device.
"""
import numpy as np
import pytest
import torch

from helpers import cos, max_rel
from oracle import momoe_oracle as orc

pytestmark = pytest.mark.gpu

CASES = {
    # headline layer: D2048 H1024 N128 K8, 16384 tokens, nothing saved
    "headline_sp0": dict(M=16384, D=2048, H=1024, N=128, K=8, Ks=0, sp=0, w_std=0.02, bias_std=0.0),
    "headline_sp100": dict(M=16384, D=2048, H=1024, N=128, K=8, Ks=0, sp=100, w_std=0.02, bias_std=0.0),
    # shared experts: 4 routed of 60 + 4 shared, 32768 tokens, half of the rows saved
    "shared_sp50": dict(M=32768, D=2048, H=1408, N=64, K=8, Ks=4, sp=50, w_std=0.02, bias_std=0.0),
    # 30B-A3B-class layer with an expert bias that unbalances the load
    "a3b_biased": dict(M=16384, D=2048, H=768, N=128, K=8, Ks=0, sp=0, w_std=0.02, bias_std=0.5),
}


@pytest.fixture(scope="module")
def momoe():
    import __graft_entry__
    __graft_entry__.build()
    torch.backends.cuda.matmul.allow_tf32 = False
    import momoe
    return momoe


@pytest.mark.parametrize("name", list(CASES))
def test_full_size_layer(momoe, name):
    from momoe import ops
    c = CASES[name]
    M, D, H, N, K, Ks, sp = c["M"], c["D"], c["H"], c["N"], c["K"], c["Ks"], c["sp"]
    dev = torch.device("cuda")
    gd = torch.Generator(device=dev).manual_seed(11)
    W1 = (torch.randn(N, D, 2 * H, generator=gd, device=dev) * c["w_std"]).bfloat16()
    W2 = (torch.randn(N, H, D, generator=gd, device=dev) * c["w_std"]).bfloat16()
    Wg = (torch.randn(D, N, generator=gd, device=dev) * c["w_std"]).bfloat16()
    x0 = torch.randn(1, M, D, generator=gd, device=dev).bfloat16()
    g0 = torch.randn(1, M, D, generator=gd, device=dev).bfloat16()
    biases = torch.cat([torch.randn(N - Ks, generator=gd, device=dev) * c["bias_std"] * 0.01,
                        torch.full((Ks,), float("-inf"), device=dev)])

    router = momoe.TopKRouter(D, N, K, Ks, Wg_DN=Wg)
    layer = momoe.MoMoE(D, H, N, K, save_percent=sp, Wl1_ND2H=W1, Wl2_NHD=W2)
    with torch.no_grad():
        _, mask_NM, s_view = router(x0, biases)
    # ---- routing, bit-exact against the reference's own torch ops on the same device
    logits = x0.reshape(M, D) @ Wg
    r = orc.router_from_logits(logits, biases, K, Ks, torch_topk=True)
    assert torch.equal(mask_NM, r["mask_NM"])
    torch.testing.assert_close(s_view, r["s_MN"].T, rtol=1e-6, atol=1e-9)
    assert int(mask_NM.sum()) == M * K and bool((mask_NM.sum(0) == K).all())

    # ---- experts with leaf x and s (an external router's view of the layer)
    x = x0.clone().requires_grad_(True)
    s = s_view.detach().clone().requires_grad_(True)
    y, sizes = layer(x, mask_NM, s)
    y.backward(g0)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(sizes, mask_NM.sum(1).to(torch.int64))
    assert torch.isfinite(y.float()).all() and torch.isfinite(x.grad.float()).all()
    y2, _ = layer(x0, mask_NM, s_view)            # forward is bitwise reproducible
    assert torch.equal(y2, y.detach())

    # ---- a subset of tokens through the CPU oracle
    sub = torch.randperm(M, generator=torch.Generator().manual_seed(3))[:40].sort().values
    W1c, W2c = W1.cpu(), W2.cpu()
    mask_sub = mask_NM[:, sub.to(dev)].cpu()
    s_sub = s_view.detach()[:, sub.to(dev)].cpu().contiguous()
    x_sub = x0[0, sub.to(dev)].cpu()
    g_sub = g0[0, sub.to(dev)].cpu()
    _, cums, idx, which = orc.permutation_from_mask(mask_sub.numpy(), K)
    y_o, fwd = orc.experts_forward(x_sub, W1c, W2c, s_sub, idx, cums, which, K)
    # save_percent only changes whether a,b are rounded to bf16 before the backward; the device rounds them either way
    gx_o, _, _, gs_o = orc.experts_backward(g_sub, x_sub, W1c, W2c, s_sub, idx, cums, which, K, 100.0, fwd,
                                            block_rows=1)
    y_d = y.detach()[0, sub.to(dev)].cpu()
    assert max_rel(y_d, y_o) <= 2e-2, "y max-rel %g" % max_rel(y_d, y_o)
    assert cos(y_d, y_o) >= 0.9999
    assert cos(x.grad[0, sub.to(dev)].cpu(), gx_o) >= 0.999
    gs_d = s.grad[:, sub.to(dev)].cpu()
    assert float(gs_d[mask_sub == 0].abs().max()) == 0.0
    assert cos(gs_d, gs_o) >= 0.999

    # ---- weight gradients of three experts against fp32 torch on the device
    for e in (0, N // 2, N - 1):
        rows = torch.nonzero(mask_NM[e]).flatten()
        if rows.numel() == 0:
            assert float(layer.Wl1_ND2H.grad[e].float().abs().sum()) == 0.0
            continue
        xs = x0[0, rows].float()
        z = xs @ W1[e].float()
        a, b = z[:, :H].bfloat16().float(), z[:, H:].bfloat16().float()
        sig = torch.sigmoid(b)
        w = s_view.detach()[e, rows][:, None]
        hh = (a * b * sig).bfloat16().float()
        gy = g0[0, rows].float()
        gh = (gy @ W2[e].float().T) * w
        gz = torch.cat([gh * b * sig, gh * a * sig * (1 + b * (1 - sig))], dim=1).bfloat16().float()
        dW2 = (hh * w).bfloat16().float().T @ gy
        dW1 = xs.T @ gz
        assert cos(layer.Wl2_NHD.grad[e], dW2) >= 0.999, (name, e)
        assert cos(layer.Wl1_ND2H.grad[e], dW1) >= 0.999, (name, e)
        assert max_rel(layer.Wl2_NHD.grad[e], dW2) <= 3e-2
        assert max_rel(layer.Wl1_ND2H.grad[e], dW1) <= 3e-2


@pytest.mark.parametrize("T", [1, 8, 64, 256, 4096])
def test_inference_token_counts(momoe, T):
    """Forward-only batches of 1..4096 tokens on the 30B-A3B-class layer (most experts receive nothing)."""
    from momoe import ops
    D, H, N, K = 2048, 768, 128, 8
    dev = torch.device("cuda")
    gd = torch.Generator(device=dev).manual_seed(5)
    W1 = (torch.randn(N, D, 2 * H, generator=gd, device=dev) * 0.02).bfloat16()
    W2 = (torch.randn(N, H, D, generator=gd, device=dev) * 0.02).bfloat16()
    x = torch.randn(1, T, D, generator=gd, device=dev).bfloat16()
    logits = (torch.randn(T, N, generator=gd, device=dev) + 0.5 * torch.randn(N, generator=gd, device=dev)).bfloat16()
    r = orc.router_from_logits(logits, torch.zeros(N, device=dev), K, 0, torch_topk=True)
    layer = momoe.MoMoE(D, H, N, K, save_percent=0, Wl1_ND2H=W1, Wl2_NHD=W2)
    with torch.no_grad():
        y, sizes = layer(x, r["mask_NM"], r["s_MN"].T)
    torch.cuda.synchronize()
    ops.check_status()
    assert int(sizes.sum()) == T * K
    sub = torch.arange(min(T, 16))
    mask_sub = r["mask_NM"][:, :len(sub)].cpu()
    _, cums, idx, which = orc.permutation_from_mask(mask_sub.numpy(), K)
    y_o, _ = orc.experts_forward(x[0, :len(sub)].cpu(), W1.cpu(), W2.cpu(), r["s_MN"].T[:, :len(sub)].cpu().contiguous(),
                                 idx, cums, which, K)
    assert max_rel(y[0, :len(sub)].cpu(), y_o) <= 2e-2
