"""`TopKRouter`: top-k softmax router with aux-loss-free bias and shared experts; same interface as the
reference (momoe/topk_router.py:151-173 there).  The gate GEMM stays a library bf16 matmul (its rounding is
part of the bit-exact selection); everything after it is one warp-per-token kernel."""
import torch
import torch.nn as nn

from . import ops
from ._lib import require_cuda


class TopKRouterFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_BSD, Wg_DN, biases_N, N, K, Ks):
        B, S, D = x_BSD.shape
        assert Wg_DN.dtype == torch.bfloat16, "Wg_DN must be of type torch.bfloat16"
        require_cuda(Wg_DN)
        dev = Wg_DN.device
        x_MD = x_BSD.reshape(B * S, D).to(device=dev, dtype=torch.bfloat16)
        Wg = Wg_DN.detach()
        with torch.cuda.device(dev):
            logits_MN = x_MD @ Wg
            topk_idx, topk_w, d = ops.route_topk(logits_MN, biases_N, K, Ks, dense=True)
        mask_NM = d["mask_NM"]
        s_NM = d["s_MN"].T
        ctx.save_for_backward(x_MD, Wg, mask_NM, d["s_postsoft_MN"], d["s_MN"], d["Ng_M"], d["Ks_M"])
        ctx.Ks = Ks
        ctx.mark_non_differentiable(mask_NM, topk_idx, topk_w)
        return x_BSD, mask_NM, s_NM, topk_idx, topk_w

    @staticmethod
    def backward(ctx, G_x_BSD, _m, G_s_NM, _i, _w):
        x_MD, Wg, mask_NM, s_postsoft_MN, s_MN, Ng_M, Ks_M = ctx.saved_tensors
        B, S, D = G_x_BSD.shape
        dev = Wg.device
        with torch.cuda.device(dev):
            G_L = ops.router_backward(G_s_NM.to(dev), s_postsoft_MN, s_MN, Ng_M, Ks_M, mask_NM, ctx.Ks)
            G_x_MD = torch.addmm(G_x_BSD.reshape(B * S, D).to(device=dev, dtype=torch.bfloat16), G_L, Wg.T)
            G_Wg = x_MD.T @ G_L
        return G_x_MD.reshape(B, S, D).to(G_x_BSD.device), G_Wg, None, None, None, None


class CompactRouterFunction(torch.autograd.Function):
    """The same router with compact outputs only: expert ids int32 [M,K] (ascending, shared experts last) and their
    weights fp32 [M,K]; the weights are the differentiable output.  No dense [N,M] tensor in either direction."""

    @staticmethod
    def forward(ctx, x_BSD, Wg_DN, biases_N, N, K, Ks):
        B, S, D = x_BSD.shape
        assert Wg_DN.dtype == torch.bfloat16, "Wg_DN must be of type torch.bfloat16"
        require_cuda(Wg_DN)
        dev = Wg_DN.device
        x_MD = x_BSD.reshape(B * S, D).to(device=dev, dtype=torch.bfloat16)
        Wg = Wg_DN.detach()
        with torch.cuda.device(dev):
            logits_MN = x_MD @ Wg
            topk_idx, topk_w, d = ops.route_topk(logits_MN, biases_N, K, Ks, dense=False, normalisers=True)
        ctx.save_for_backward(x_MD, Wg, topk_idx, topk_w, d["Ng_M"], d["Ks_M"])
        ctx.dims = (B, S, D, N, Ks)
        ctx.x_device = x_BSD.device
        ctx.mark_non_differentiable(topk_idx)
        return topk_idx, topk_w

    @staticmethod
    def backward(ctx, _i, G_w_MK):
        x_MD, Wg, topk_idx, topk_w, Ng_M, Ks_M = ctx.saved_tensors
        B, S, D, N, Ks = ctx.dims
        dev = Wg.device
        with torch.cuda.device(dev):
            G_L = ops.router_backward_from_topk_grad(G_w_MK.to(dev), topk_idx, topk_w, Ng_M, Ks_M, N, Ks)
            G_x_MD = G_L @ Wg.T
            G_Wg = x_MD.T @ G_L
        return G_x_MD.reshape(B, S, D).to(ctx.x_device), G_Wg, None, None, None, None


class TopKRouter(nn.Module):
    def __init__(self, embedding_dim, num_experts, num_chosen_experts, num_shared_experts,
                 Wg_DN: torch.Tensor | None = None):
        super().__init__()
        self.D = embedding_dim
        self.N = num_experts
        self.K = num_chosen_experts
        self.Ks = num_shared_experts
        if Wg_DN is None:
            self.Wg_DN = nn.Parameter(torch.randn((self.D, self.N), device="cuda", dtype=torch.bfloat16) / self.D,
                                      requires_grad=True)
        else:
            self.Wg_DN = nn.Parameter(Wg_DN.clone().detach().to(torch.bfloat16), requires_grad=True)

    def forward(self, x_BSD, biases_N):
        x_BSD, mask_NM, s_NM, topk_idx, topk_w = TopKRouterFunction.apply(x_BSD, self.Wg_DN, biases_N, self.N,
                                                                          self.K, self.Ks)
        # the compact form of the same routing rides along so that MoMoE need not re-derive it from the mask
        from .momoe import attach_compact_routing
        attach_compact_routing(mask_NM, s_NM, topk_idx, topk_w)
        return x_BSD, mask_NM, s_NM
