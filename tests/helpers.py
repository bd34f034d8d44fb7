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
