"""`MoE`: router + MoMoE + aux-loss-free bias update, same interface as the reference wrapper
(momoe/sample_moe.py:16-68 there).

By default the wrapper runs router and experts as one autograd node that keeps the routing in its compact form
(top-k ids, weights, permutation): the dense `mask_NM` / `s_NM` of the two-module composition, the dense `G_s_NM` and
the dense router backward are never materialised.  `MoE.fused = False` restores the literal composition
`TopKRouter -> MoMoE`; both give the same output bit for bit."""
import torch
import torch.nn as nn

from . import ops
from ._lib import require_cuda
from .momoe import MoMoE, _CHECK
from .topk_router import TopKRouter


class FusedMoEFunction(torch.autograd.Function):
    """Gate GEMM -> router kernel -> permutation -> experts, and the matching backward, on compact routing data.
    Stands in for momoe/topk_router.py:85-145 plus momoe/momoe.py:847-903 of the reference."""

    @staticmethod
    def forward(ctx, x_BSD, Wg_DN, Wl1_ND2H, Wl2_NHD, biases_N, K, Ks, save_percent):
        B, S, D = x_BSD.shape
        assert Wg_DN.dtype == torch.bfloat16, "Wg_DN must be of type torch.bfloat16"
        assert Wl1_ND2H.device == Wl2_NHD.device, \
            "All weights must be on the same device, but got: Wl1_ND2H.device = {}, Wl2_NHD.device = {}".format(
                Wl1_ND2H.device, Wl2_NHD.device)
        require_cuda(Wl1_ND2H, Wg_DN)
        dev = Wl1_ND2H.device
        N, H, _ = Wl2_NHD.shape
        x_MD = x_BSD.reshape(B * S, D).to(device=dev, dtype=torch.bfloat16).contiguous()
        Wg = Wg_DN.detach()
        W1 = Wl1_ND2H.detach().to(torch.bfloat16).contiguous()
        W2 = Wl2_NHD.detach().to(torch.bfloat16).contiguous()
        with torch.cuda.device(dev):
            logits_MN = x_MD @ Wg
            topk_idx, topk_w, d = ops.route_topk(logits_MN, biases_N, K, Ks, dense=False, normalisers=True)
            plan = ops.RoutingPlan.from_topk(topk_idx, topk_w, N, D, H, save_percent)
            y_MD, a_save, b_save = ops.experts_forward(plan, x_MD, W1, W2,
                                                          inference=not any(ctx.needs_input_grad))
        ctx.plan = plan
        ctx.shape = (B, S, D)
        ctx.Ks = Ks
        ctx.x_device = x_BSD.device
        saved = [x_MD, Wg, W1, W2, d["Ng_M"], d["Ks_M"]]
        ctx.has_ab = a_save is not None
        if ctx.has_ab:
            saved += [a_save, b_save]
        ctx.save_for_backward(*saved)
        ctx.mark_non_differentiable(plan.sizes)
        ops.status_post(dev)
        if _CHECK:
            ops.check_status(dev)
        return y_MD.reshape(B, S, D).to(device=x_BSD.device), plan.sizes

    @staticmethod
    def backward(ctx, G_y_BSD, _):
        saved = ctx.saved_tensors
        x_MD, Wg, W1, W2, Ng_M, Ks_M = saved[:6]
        a_save, b_save = (saved[6], saved[7]) if ctx.has_ab else (None, None)
        B, S, D = ctx.shape
        plan = ctx.plan
        dev = W1.device
        g_MD = G_y_BSD.reshape(B * S, D).to(device=dev, dtype=torch.bfloat16).contiguous()
        with torch.cuda.device(dev):
            G_x, G_W1, G_W2, gs_part = ops.experts_backward(plan, g_MD, x_MD, W1, W2, a_save, b_save,
                                                            need_gs_dense=False)
            G_L = ops.router_backward_compact(plan, gs_part, Ng_M, Ks_M, ctx.Ks)
            G_x = torch.addmm(G_x, G_L, Wg.T)
            G_Wg = x_MD.T @ G_L
        ops.status_post(dev)
        if _CHECK:
            ops.check_status(dev)
        return G_x.reshape(B, S, D).to(ctx.x_device), G_Wg, G_W1, G_W2, None, None, None, None


class MoE(nn.Module):
    def __init__(self, embedding_dim, intermediate_dim, num_experts, num_chosen_experts, num_shared_experts,
                 save_percent=0, bias_update_rate=1e-4, Wg_DN: torch.Tensor | None = None,
                 Wl1_ND2H: torch.Tensor | None = None, Wl2_NHD: torch.Tensor | None = None):
        super().__init__()
        self.D = embedding_dim
        self.H = intermediate_dim
        self.N = num_experts
        self.K = num_chosen_experts
        self.Ks = num_shared_experts
        self.save_percent = save_percent
        self.bias_update_rate = bias_update_rate
        self.router = TopKRouter(embedding_dim=self.D, num_experts=self.N, num_chosen_experts=self.K,
                                 num_shared_experts=self.Ks, Wg_DN=Wg_DN)
        self.momoe = MoMoE(embedding_dim=self.D, intermediate_dim=self.H, num_experts=self.N,
                           num_chosen_experts=self.K, save_percent=self.save_percent, Wl1_ND2H=Wl1_ND2H,
                           Wl2_NHD=Wl2_NHD)
        dev = self.momoe.Wl1_ND2H.device
        self.biases_N = nn.Parameter(
            torch.cat([torch.zeros(self.N - self.Ks, device=dev, dtype=torch.float32),
                       torch.full((self.Ks,), float("-inf"), device=dev, dtype=torch.float32)], dim=-1),
            requires_grad=False)
        self.fused = True

    def forward(self, x_BSD):
        if self.fused:
            ops.status_poll(self.momoe.Wl1_ND2H.device)  # raises if an earlier pass left a device-side error code
            y_BSD, sizes_N = FusedMoEFunction.apply(x_BSD, self.router.Wg_DN, self.momoe.Wl1_ND2H,
                                                    self.momoe.Wl2_NHD, self.biases_N, self.K, self.Ks,
                                                    self.save_percent)
        else:
            x_BSD, mask_NM, s_NM = self.router(x_BSD, self.biases_N)
            y_BSD, sizes_N = self.momoe(x_BSD, mask_NM, s_NM)
        # DeepSeek-style auxiliary-loss-free balancing: push the bias of under-loaded experts up
        B, S, _ = x_BSD.shape
        c_avg = B * S * (self.K - self.Ks) / (self.N - self.Ks)
        with torch.no_grad():
            ops.bias_update_(self.biases_N.data, sizes_N, self.Ks, c_avg, self.bias_update_rate)
        return y_BSD
