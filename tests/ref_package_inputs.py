"""Seeded inputs shared by the reference-package worker and the test that compares against it."""
import torch

CASES = {
    "mid_shared_sp50": dict(B=2, S=512, D=512, H=256, N=16, K=4, Ks=1, sp=50, bias_std=0.01),
    "chart_c1": dict(B=2, S=512, D=1024, H=512, N=32, K=4, Ks=0, sp=0, bias_std=0.0),
    "ragged_sp100": dict(B=1, S=777, D=384, H=192, N=12, K=3, Ks=0, sp=100, bias_std=0.02),
}


def make_inputs(c):
    g = torch.Generator().manual_seed(c["D"] + c["N"])
    N, D, H, Ks = c["N"], c["D"], c["H"], c["Ks"]
    return dict(
        x=torch.randn(c["B"], c["S"], D, generator=g).bfloat16(),
        g=torch.randn(c["B"], c["S"], D, generator=g).bfloat16(),
        W1=(torch.randn(N, D, 2 * H, generator=g) * 0.03).bfloat16(),
        W2=(torch.randn(N, H, D, generator=g) * 0.03).bfloat16(),
        Wg=(torch.randn(D, N, generator=g) * 0.03).bfloat16(),
        biases=torch.cat([torch.randn(N - Ks, generator=g) * c["bias_std"], torch.full((Ks,), float("-inf"))]))
