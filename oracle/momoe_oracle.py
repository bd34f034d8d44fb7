"""CPU restatement of the reference MoMoE layer (router -> permutation -> SwiGLU experts -> combine)
and of its backward pass.

THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke check and the
`cpu_baseline` / `--impl reference` legs of the benchmark may import it; the product path never does.

Parity status: pinned.  Every function here is checked against fixtures produced by running the
reference's own kernels (Triton interpreter on CPU) on seeded inputs; the fixtures and the script that
made them live in `tests/golden/`.

Every rounding point of the reference is reproduced: the arithmetic is fp32 on bf16-valued operands and
results are rounded to bf16 exactly where the reference rounds them.  Functions cite the reference lines
they restate (paths are relative to the reference project root).
"""
from __future__ import annotations

import numpy as np
import torch

bf16 = torch.bfloat16
f32 = torch.float32


def _r(t: torch.Tensor) -> torch.Tensor:
    """Round an fp32 tensor to bf16 and return it as fp32 (one bf16 rounding point)."""
    return t.to(bf16).to(f32)


# ----------------------------------------------------------------------------------------------------
# Router
# ----------------------------------------------------------------------------------------------------
def topk_lowest_index_first(score_MN: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest entries per row; among equal values the lowest index wins.

    This is the selection rule of the CUDA `torch.topk` the reference calls (momoe/topk_router.py:101):
    a radix select finds the k-th value, then entries strictly greater are taken, then entries equal to
    it in index order.  Returned indices are sorted ascending (only the set matters to the reference).
    NaNs are not expected (softmax of finite logits plus finite bias).
    """
    order = torch.sort(score_MN, dim=-1, descending=True, stable=True).indices[:, :k]
    return torch.sort(order, dim=-1).values


def gate_logits(x_MD: torch.Tensor, Wg_DN: torch.Tensor) -> torch.Tensor:
    """bf16-rounded gate logits, momoe/topk_router.py:92-95 (fp32 accumulate, bf16 output)."""
    return (x_MD.to(bf16).to(f32) @ Wg_DN.to(bf16).to(f32)).to(bf16)


def router_from_logits(logits_MN: torch.Tensor, biases_N: torch.Tensor, K: int, Ks: int, torch_topk: bool = False):
    """Everything in momoe/topk_router.py:96-120 after the gate GEMM.

    Runs on the device of `logits_MN`.  With `torch_topk=True` the selection is `torch.topk` itself, i.e. on a
    CUDA tensor exactly the call the reference makes; otherwise the documented tie rule is applied explicitly.

    logits_MN: bf16 [M, N].  biases_N: fp32 [N] (entries of shared experts are ignored).
    Returns dict with
      mask_NM int32 [N, M] contiguous (all ones on the last Ks rows)      (:110-119)
      s_MN fp32 [M, N] normalised weights (s_NM of the reference is its transpose view, :120)
      s_postsoft_MN fp32 [M, N] masked probabilities before renormalisation  (:106)
      Ng_M, Ks_M fp32 [M]                                                 (:104-105)
      topk_idx int32 [M, K] ascending expert ids of the selected + shared experts
    """
    M, N = logits_MN.shape
    dev = logits_MN.device
    Ng = N - Ks
    p_g = torch.softmax(logits_MN[:, :Ng], dim=-1, dtype=f32)
    s_MN = torch.empty((M, N), dtype=f32, device=dev)
    if Ks > 0:
        p_s = torch.softmax(logits_MN[:, Ng:], dim=-1, dtype=f32)
    else:
        p_s = torch.empty((M, 0), dtype=f32, device=dev)
    score = p_g + biases_N.to(dev)[:Ng].to(f32)[None, :]
    if torch_topk:
        sel = torch.sort(torch.topk(score, K - Ks, dim=-1).indices, dim=-1).values
    else:
        sel = topk_lowest_index_first(score, K - Ks)
    mask_MNg = torch.zeros((M, Ng), dtype=torch.bool, device=dev)
    mask_MNg.scatter_(1, sel, True)
    q = p_g * mask_MNg
    Ng_M = q.sum(dim=-1)
    Ks_M = p_s.sum(dim=-1)
    s_postsoft = torch.cat([q, p_s], dim=-1)
    s_MN[:, :Ng] = q / Ng_M[:, None]
    s_MN[:, Ng:] = p_s / Ks_M[:, None]
    mask_NM = torch.ones((N, M), dtype=torch.int32, device=dev)
    mask_NM[:Ng] = mask_MNg.T.to(torch.int32)
    shared = torch.arange(Ng, N, dtype=sel.dtype, device=dev)[None, :].expand(M, Ks)
    topk_idx = torch.cat([sel, shared], dim=-1).to(torch.int32)
    return dict(mask_NM=mask_NM.contiguous(), s_MN=s_MN, s_postsoft_MN=s_postsoft, Ng_M=Ng_M, Ks_M=Ks_M,
                topk_idx=topk_idx)


def router_backward(G_s_NM, s_postsoft_MN, s_MN, Ng_M, Ks_M, mask_NM, Ks, x_MD, Wg_DN, G_x_MD):
    """momoe/topk_router.py:11-56 (renormalisation + softmax backward, bf16 store) and :139-141
    (`G_x += G_L @ Wg^T`, `G_Wg = x^T @ G_L`, both bf16 GEMMs)."""
    N, M = G_s_NM.shape
    Ng = N - Ks
    G = G_s_NM.T.to(f32)
    msk = mask_NM.T.to(f32)
    out = torch.zeros((M, N), dtype=f32)
    # gating group: mask applies to the first dot product only (:39)
    dot_g = (G[:, :Ng] * s_MN[:, :Ng] * msk[:, :Ng]).sum(-1, keepdim=True)
    u_g = (G[:, :Ng] - dot_g) * (1.0 / Ng_M)[:, None]
    t_g = (u_g * s_postsoft_MN[:, :Ng]).sum(-1, keepdim=True)
    out[:, :Ng] = s_postsoft_MN[:, :Ng] * (u_g - t_g)
    if Ks > 0:
        dot_s = (G[:, Ng:] * s_MN[:, Ng:]).sum(-1, keepdim=True)
        u_s = (G[:, Ng:] - dot_s) * (1.0 / Ks_M)[:, None]
        t_s = (u_s * s_postsoft_MN[:, Ng:]).sum(-1, keepdim=True)
        out[:, Ng:] = s_postsoft_MN[:, Ng:] * (u_s - t_s)
    G_L = _r(out)                                                     # :51-52, :136 (.to(bf16))
    G_x = _r(_r(G_x_MD.to(f32)) + G_L @ Wg_DN.to(f32).T)              # :139 addmm in bf16
    G_Wg = _r(x_MD.to(bf16).to(f32).T @ G_L)                          # :141
    return G_x.to(bf16), G_Wg.to(bf16), G_L.to(bf16)


# ----------------------------------------------------------------------------------------------------
# Permutation (integers; numpy)
# ----------------------------------------------------------------------------------------------------
def permutation_from_mask(mask_NM: np.ndarray, K: int):
    """momoe/momoe.py:821-842 and the kernel at :760-815.

    sizes_N int64 [N]; cumsums_N int32 [N+1] (exclusive scan, last entry forced to M*K, :792-793);
    idx_Msum int32 [M*K] = token ids, expert-major, ascending inside an expert (== nonzero(mask)[:, 1]);
    which_Msum int32 [M*K] = slot 0..K-1 of that (token, expert) pair.  The reference hands slots out with
    an atomic counter (:812) so any bijection per token is valid; the canonical choice here is the rank
    of the expert among the token's experts in ascending id, which is what sequential execution gives.
    """
    mask = np.asarray(mask_NM) != 0
    N, M = mask.shape
    sizes = mask.sum(axis=1).astype(np.int64)
    cumsums = np.zeros(N + 1, dtype=np.int32)
    cumsums[1:] = np.cumsum(sizes).astype(np.int32)
    cumsums[N] = M * K
    e_ids, idx = np.nonzero(mask)
    slot_dense = np.cumsum(mask, axis=0) - 1          # rank of expert e among token m's experts
    which = slot_dense[e_ids, idx].astype(np.int32)
    return sizes, cumsums, idx.astype(np.int32), which


# ----------------------------------------------------------------------------------------------------
# Experts forward / backward
# ----------------------------------------------------------------------------------------------------
def save_rows(Msum: int, save_percent: float) -> int:
    """momoe/momoe.py:251."""
    return int(Msum * save_percent / 100.0)


def experts_forward(x_MD, W1_ND2H, W2_NHD, s_NM, idx, cumsums, which, K):
    """momoe/momoe.py:108-152 (up/gate + SwiGLU), :200-237 (down, weight, slab scatter), :290 (sum over K).

    Returns y_MD bf16 and the intermediates a, b (fp32, unrounded), h (bf16-valued fp32) and
    ypre (fp32) in expert-major row order.
    """
    x = x_MD.to(bf16).to(f32)
    W1 = W1_ND2H.to(bf16).to(f32)
    W2 = W2_NHD.to(bf16).to(f32)
    M, D = x.shape
    N, H, _ = W2.shape
    Msum = int(cumsums[-1])
    a = torch.zeros((Msum, H), dtype=f32)
    b = torch.zeros((Msum, H), dtype=f32)
    h = torch.zeros((Msum, H), dtype=f32)
    ypre = torch.zeros((Msum, D), dtype=f32)
    Y = torch.zeros((K, M, D), dtype=f32)
    idx_t = torch.as_tensor(np.asarray(idx), dtype=torch.long)
    which_t = torch.as_tensor(np.asarray(which), dtype=torch.long)
    for e in range(N):
        lo, hi = int(cumsums[e]), int(cumsums[e + 1])
        if hi == lo:
            continue
        rows = idx_t[lo:hi]
        z = x[rows] @ W1[e]
        a[lo:hi], b[lo:hi] = z[:, :H], z[:, H:]
        h[lo:hi] = _r(b[lo:hi] * torch.sigmoid(b[lo:hi]) * a[lo:hi])          # :148
        ypre[lo:hi] = h[lo:hi] @ W2[e]                                          # :217
        w = s_NM[e].to(f32)[rows]
        Y[which_t[lo:hi], rows] = _r(ypre[lo:hi] * w[:, None])                  # :235-237
    y = Y.sum(dim=0).to(bf16)                                                   # :290
    return y, dict(a=a, b=b, h=h, ypre=ypre)


def experts_backward(G_y_MD, x_MD, W1_ND2H, W2_NHD, s_NM, idx, cumsums, which, K, save_percent,
                     fwd, block_rows=128):
    """momoe/momoe.py:298-350 (gathers), :421-535 (dgrad-2 + SwiGLU'), :356-412 (wgrads),
    :612-703 (dgrad-1, G_s), :754 (sum over K).

    `fwd` is the dict returned by `experts_forward`.  Tiles lying entirely below
    Msave = int(Msum * save_percent / 100) use the bf16-rounded saved a, b, ypre (:486-491, :685-688);
    others use the unrounded recomputation (:492-515, :689-697).  `block_rows` is the reference's
    BLOCK_SIZE_Mi (128 in its first tile configuration).
    Returns G_x bf16 [M, D], G_W1 bf16, G_W2 bf16, G_s_NM fp32 [N, M] (zero where unselected).
    """
    g = G_y_MD.to(bf16).to(f32)
    x = x_MD.to(bf16).to(f32)
    W1 = W1_ND2H.to(bf16).to(f32)
    W2 = W2_NHD.to(bf16).to(f32)
    M, D = x.shape
    N, H, _ = W2.shape
    Msum = int(cumsums[-1])
    Msave = save_rows(Msum, save_percent)
    idx_t = torch.as_tensor(np.asarray(idx), dtype=torch.long)
    which_t = torch.as_tensor(np.asarray(which), dtype=torch.long)
    G_W1 = torch.zeros_like(W1)
    G_W2 = torch.zeros_like(W2)
    G_s = torch.zeros((N, M), dtype=f32)
    GX = torch.zeros((K, M, D), dtype=f32)
    for e in range(N):
        lo, hi = int(cumsums[e]), int(cumsums[e + 1])
        if hi == lo:
            continue
        rows = idx_t[lo:hi]
        w = s_NM[e].to(f32)[rows]
        gy = _r(g[rows] * w[:, None])                                           # :340
        xs = x[rows]
        Gh = gy @ W2[e].T                                                        # :474-480
        a = fwd["a"][lo:hi].clone()
        b = fwd["b"][lo:hi].clone()
        # tile-granular rule: a row uses saved (bf16-rounded) values iff its whole tile lies below Msave
        t0 = lo + ((torch.arange(lo, hi) - lo) // block_rows) * block_rows
        saved = (t0 + block_rows) <= Msave
        a[saved] = _r(a[saved])
        b[saved] = _r(b[saved])
        sig = torch.sigmoid(b)
        Gz = _r(torch.cat([Gh * b * sig, Gh * a * sig * (1 + b * (1 - sig))], dim=1))   # :524-530
        hh = _r(a * b * sig)                                                     # :533-535
        G_W2[e] = _r(hh.T @ gy)                                                  # :593-600, :412
        G_W1[e] = _r(xs.T @ Gz)                                                  # :730-737
        GX[which_t[lo:hi], rows] = _r(Gz @ W1[e].T)                              # :666-681
        ypre = hh @ W2[e]                                                        # :689-697 (recompute)
        ypre[saved] = _r(fwd["ypre"][lo:hi][saved])                              # :685-688 (saved bf16)
        G_s[e, rows] = (g[rows] * ypre).sum(dim=1)                               # :699-703
    G_x = GX.sum(dim=0).to(bf16)                                                 # :754
    return G_x, G_W1.to(bf16), G_W2.to(bf16), G_s


# ----------------------------------------------------------------------------------------------------
# Wrapper
# ----------------------------------------------------------------------------------------------------
def bias_update(biases_N, sizes_N, M, K, Ks, rate):
    """momoe/sample_moe.py:63-66."""
    N = biases_N.shape[0]
    c_avg = M * (K - Ks) / (N - Ks)
    return biases_N + rate * torch.sign(c_avg - torch.as_tensor(sizes_N).to(f32))


def moe_forward_backward(x_BSD, Wg_DN, W1_ND2H, W2_NHD, biases_N, K, Ks, save_percent=0.0,
                         G_y_BSD=None, loss="sumsq", block_rows=128, logits=None):
    """Whole layer as momoe/sample_moe.py:59-68 composes it, followed by the backward of
    `loss = sum(y.float()**2)` (or an explicit upstream gradient).  Returns a dict of every
    observable tensor.  `logits` (bf16 [M,N]) replaces the gate GEMM's output (momoe/topk_router.py:95):
    a caller that compares against a device run passes the logits the device's library GEMM produced, whose
    bf16 rounding may differ from the CPU GEMM's in the last bit."""
    B, S, D = x_BSD.shape
    M = B * S
    N = W2_NHD.shape[0]
    x_MD = x_BSD.reshape(M, D)
    if logits is None:
        logits = gate_logits(x_MD, Wg_DN)
    r = router_from_logits(logits, biases_N, K, Ks)
    sizes, cumsums, idx, which = permutation_from_mask(r["mask_NM"].numpy(), K)
    s_NM = r["s_MN"].T
    y, fwd = experts_forward(x_MD, W1_ND2H, W2_NHD, s_NM, idx, cumsums, which, K)
    out = dict(logits=logits, sizes=sizes, cumsums=cumsums, idx=idx, which=which, y=y.reshape(B, S, D),
               new_biases=bias_update(biases_N, sizes, M, K, Ks, 1e-4), **r)
    if G_y_BSD is None and loss is None:
        return out
    if G_y_BSD is None:
        G_y = 2.0 * y.to(f32)
    else:
        G_y = G_y_BSD.reshape(M, D).to(f32)
    G_x, G_W1, G_W2, G_s = experts_backward(G_y, x_MD, W1_ND2H, W2_NHD, s_NM, idx, cumsums, which, K,
                                            save_percent, fwd, block_rows)
    G_x2, G_Wg, G_L = router_backward(G_s, r["s_postsoft_MN"], r["s_MN"], r["Ng_M"], r["Ks_M"],
                                      r["mask_NM"], Ks, x_MD, Wg_DN, G_x)
    out.update(G_x_experts=G_x, G_W1=G_W1, G_W2=G_W2, G_s_NM=G_s, G_x=G_x2.reshape(B, S, D), G_Wg=G_Wg,
               G_L=G_L)
    return out


# ----------------------------------------------------------------------------------------------------
# Throughput-oriented variant for the CPU baseline timing (same math, autograd backward)
# ----------------------------------------------------------------------------------------------------
def cpu_baseline_prepare(Wg_DN, W1_ND2H, W2_NHD):
    """fp32 per-expert leaf weights (views of one buffer, so a gradient is only materialised for experts that
    received tokens).  Done once, outside the timed region."""
    W1 = W1_ND2H.to(f32)
    W2 = W2_NHD.to(f32)
    return dict(Wg=Wg_DN.to(f32).requires_grad_(True),
                W1=[w.detach().requires_grad_(True) for w in W1.unbind(0)],
                W2=[w.detach().requires_grad_(True) for w in W2.unbind(0)])


def cpu_baseline_step(state, x_BSD, biases_N, K, Ks):
    """One fwd+bwd of the layer on the host cores: sparse per-expert index_select -> matmuls -> SiLU*mul ->
    matmul -> index_add_, autograd for the backward, all available torch threads.  Follows
    momoe/sample_moe.py:59-68 and the math of momoe/momoe.py; used only as the timed CPU baseline."""
    B, S, D = x_BSD.shape
    M = B * S
    W1, W2, Wg = state["W1"], state["W2"], state["Wg"]
    N = len(W1)
    H = W2[0].shape[0]
    for w in W1 + W2 + [Wg]:
        w.grad = None
    x = x_BSD.reshape(M, D).to(f32).requires_grad_(True)
    raw = x @ Wg
    Ng = N - Ks
    p = torch.softmax(raw[:, :Ng], dim=-1)
    sel = torch.topk(p.detach() + biases_N[:Ng][None, :], K - Ks, dim=-1).indices
    q = torch.gather(p, 1, sel)
    w_sel = q / q.sum(-1, keepdim=True)
    flat_e = sel.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    counts = torch.bincount(flat_e, minlength=Ng)
    tok = order // (K - Ks)
    wflat = w_sel.reshape(-1)[order]
    parts, rows_all = [], []
    start = 0
    for e in range(Ng):
        c = int(counts[e])
        if c == 0:
            continue
        rows = tok[start:start + c]
        z = x.index_select(0, rows) @ W1[e]
        hh = z[:, :H] * torch.nn.functional.silu(z[:, H:])
        parts.append((hh @ W2[e]) * wflat[start:start + c, None])
        rows_all.append(rows)
        start += c
    y = torch.zeros((M, D), dtype=f32).index_add(0, torch.cat(rows_all), torch.cat(parts))
    if Ks > 0:
        ps = torch.softmax(raw[:, Ng:], dim=-1)
        for j in range(Ks):
            z = x @ W1[Ng + j]
            hh = z[:, :H] * torch.nn.functional.silu(z[:, H:])
            y = y + (hh @ W2[Ng + j]) * ps[:, j:j + 1]
    loss = (y ** 2).sum()
    loss.backward()
    return loss.detach(), counts
