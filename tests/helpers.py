"""Shared helpers for the parity tests: golden fixture loading and the parity metrics."""
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def from_bits(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    g = {}
    for k in z.files:
        if k.endswith("_bf16"):
            g[k[:-5]] = from_bits(z[k])
        elif k in ("meta", "save_percent"):
            g[k] = z[k]
        else:
            g[k] = torch.from_numpy(z[k])
    B, S, D, H, N, K, Ks, block_rows = [int(v) for v in g["meta"]]
    g.update(B=B, S=S, D=D, H=H, N=N, K=K, Ks=Ks, block_rows=block_rows, sp=float(g["save_percent"]))
    return g


def cos(a, b):
    a = a.double().flatten()
    b = b.double().flatten()
    na, nb = a.norm(), b.norm()
    if na == 0 and nb == 0:
        return 1.0
    return float((a @ b) / (na * nb))


def max_rel(a, b):
    """max |a-b| / max |b|: the elementwise error relative to the reference tensor's scale."""
    a = a.double()
    b = b.double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


# ---------------------------------------------------------------------------------------------------------
# GPU-side helpers
# ---------------------------------------------------------------------------------------------------------
def make_routing(M, N, K, seed, skew=0.0, device="cuda"):
    """Seeded random routing: topk_idx int32 [M,K] ascending, topk_w fp32 [M,K] summing to 1 per token."""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(M, N, generator=g) + skew * torch.randn(N, generator=g)[None, :]
    idx = torch.sort(torch.topk(logits, K, dim=-1).indices, dim=-1).values.to(torch.int32)
    w = torch.softmax(torch.gather(logits, 1, idx.long()), dim=-1).float()
    return idx.to(device), w.to(device)


def dense_from_topk(topk_idx, topk_w, N):
    M, K = topk_idx.shape
    mask = torch.zeros((M, N), dtype=torch.int32, device=topk_idx.device)
    mask.scatter_(1, topk_idx.long(), 1)
    s = torch.zeros((M, N), dtype=torch.float32, device=topk_idx.device)
    s.scatter_(1, topk_idx.long(), topk_w)
    return mask.T.contiguous(), s.T   # s_NM as a transposed view, like the reference router returns it


def expert_rows(plan):
    """Host copies of the plan tables: list of (expert, first padded row, count, token ids, weights)."""
    cum = plan.cumsums.cpu().numpy()
    pad = plan.pad_off.cpu().numpy()
    idx = plan.idx.cpu()
    out = []
    for e in range(plan.N):
        c = int(cum[e + 1] - cum[e])
        out.append((e, int(pad[e]), c, idx[int(cum[e]):int(cum[e + 1])].long()))
    return out
