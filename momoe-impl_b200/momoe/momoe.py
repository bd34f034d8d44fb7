"""`MoMoE`: the memory-optimised SwiGLU mixture-of-experts layer, same constructor, parameters and
`(y_BSD, tokens_per_expert_N)` contract as the reference module (momoe/momoe.py:914-972 there), running on
hand-written sm_100a kernels through libmomoe_b200.so."""
import os

import torch
import torch.nn as nn

from . import ops
from ._lib import require_cuda


# MOMOE_B200_CHECK=1: synchronise after every forward / backward and raise if a kernel reported a device-side problem
# (a token without exactly K experts, a wait that ran out).  Off by default: the layer never synchronises the host.
_CHECK = os.environ.get("MOMOE_B200_CHECK", "0") == "1"


def attach_compact_routing(mask_NM, s_NM, topk_idx, topk_w):
    """Let the dense router outputs carry the compact form of the same routing (ids and weights [M,K]), so that
    `MoMoE` need not re-derive it from the mask.  The tag records both tensors' version counters."""
    tag = (topk_idx, topk_w, mask_NM._version, s_NM._version)
    mask_NM._momoe_topk = tag
    s_NM._momoe_topk = tag


def compact_routing_of(mask_NM, s_NM):
    """The compact routing attached by `TopKRouter`, or None.  It is only trusted when BOTH tensors passed in are
    the very objects the router returned and neither has been written since: a caller that rescales `s_NM`, passes
    other weights, or edits `mask_NM` in place (the reference reads whatever it is given, momoe/momoe.py:235-237,
    760-815) gets the routing re-derived from the dense tensors."""
    tag = getattr(mask_NM, "_momoe_topk", None)
    if tag is None or getattr(s_NM, "_momoe_topk", None) is not tag:
        return None
    if mask_NM._version != tag[2] or s_NM._version != tag[3]:
        return None
    return tag[0], tag[1]


class MoEFunction(torch.autograd.Function):
    """Forward / backward orchestration; stands in for momoe/momoe.py:847-903 of the reference."""

    @staticmethod
    def forward(ctx, x_BSD, Wl1_ND2H, Wl2_NHD, mask_NM, s_NM, K, save_percent):
        B, S, D = x_BSD.shape
        assert Wl1_ND2H.device == Wl2_NHD.device, \
            "All weights must be on the same device, but got: Wl1_ND2H.device = {}, Wl2_NHD.device = {}".format(
                Wl1_ND2H.device, Wl2_NHD.device)
        dev = Wl1_ND2H.device
        require_cuda(Wl1_ND2H)
        N, H, _ = Wl2_NHD.shape
        x_MD = x_BSD.reshape(B * S, D).to(device=dev, dtype=torch.bfloat16).contiguous()
        W1 = Wl1_ND2H.detach().to(torch.bfloat16).contiguous()
        W2 = Wl2_NHD.detach().to(torch.bfloat16).contiguous()
        with torch.cuda.device(dev):
            compact = compact_routing_of(mask_NM, s_NM)
            if compact is not None and compact[0].shape == (B * S, K):
                plan = ops.RoutingPlan.from_topk(compact[0], compact[1], N, D, H, save_percent)
            else:
                plan = ops.RoutingPlan.from_mask(mask_NM.to(dev), s_NM.to(dev), K, D, H, save_percent)
            y_MD, a_save, b_save = ops.experts_forward(plan, x_MD, W1, W2,
                                                          inference=not any(ctx.needs_input_grad))
        ctx.plan = plan
        ctx.shape = (B, S, D)
        ctx.in_devices = (x_BSD.device, s_NM.device)
        saved = [x_MD, W1, W2]
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
        x_MD, W1, W2 = saved[:3]
        a_save, b_save = (saved[3], saved[4]) if ctx.has_ab else (None, None)
        B, S, D = ctx.shape
        plan = ctx.plan
        dev = W1.device
        g_MD = G_y_BSD.reshape(B * S, D).to(device=dev, dtype=torch.bfloat16).contiguous()
        with torch.cuda.device(dev):
            G_x, G_W1, G_W2, G_s = ops.experts_backward(plan, g_MD, x_MD, W1, W2, a_save, b_save)
        ops.status_post(dev)
        if _CHECK:
            ops.check_status(dev)
        x_dev, s_dev = ctx.in_devices
        return G_x.reshape(B, S, D).to(x_dev), G_W1, G_W2, None, G_s.to(s_dev), None, None


class MoMoE(nn.Module):
    def __init__(self, embedding_dim, intermediate_dim, num_experts, num_chosen_experts, save_percent=0,
                 Wl1_ND2H: torch.Tensor | None = None, Wl2_NHD: torch.Tensor | None = None):
        """
        Args:
            embedding_dim: input / output width D.
            intermediate_dim: hidden width H of each expert.
            num_experts: N.
            num_chosen_experts: experts per token K (shared experts included).
            save_percent: share (0..100) of the expert-major rows whose pre-activations are kept for backward;
                the rest is recomputed.
            Wl1_ND2H: up/gate weights [N, D, 2H] (columns [:H] linear half, [H:] gated half), or None.
            Wl2_NHD: down weights [N, H, D], or None.
        """
        assert save_percent >= 0 and save_percent <= 100, \
            "save_percent must be between 0 and 100 inclusive, got {}".format(save_percent)
        super().__init__()
        self.D = embedding_dim
        self.H = intermediate_dim
        self.N = num_experts
        self.K = num_chosen_experts
        self.save_percent = save_percent
        if Wl1_ND2H is None:
            self.Wl1_ND2H = nn.Parameter(
                torch.randn((self.N, self.D, 2 * self.H), device="cuda", dtype=torch.bfloat16) / self.D,
                requires_grad=True)
        else:
            self.Wl1_ND2H = nn.Parameter(Wl1_ND2H.clone().detach().to(torch.bfloat16), requires_grad=True)
        if Wl2_NHD is None:
            self.Wl2_NHD = nn.Parameter(
                torch.randn((self.N, self.H, self.D), device="cuda", dtype=torch.bfloat16) / self.D,
                requires_grad=True)
        else:
            self.Wl2_NHD = nn.Parameter(Wl2_NHD.clone().detach().to(torch.bfloat16), requires_grad=True)

    def forward(self, x_BSD, mask_NM, s_NM):
        """x_BSD [B,S,D]; mask_NM int32 [N,M] of 0/1 with exactly K ones per token; s_NM [N,M] routing weights
        (zero where unselected).  Returns (y_BSD bf16, tokens_per_expert_N int64)."""
        ops.status_poll(self.Wl1_ND2H.device)      # raises if an earlier pass left a device-side error code
        y_BSD, sizes_N = MoEFunction.apply(x_BSD, self.Wl1_ND2H, self.Wl2_NHD, mask_NM, s_NM, self.K,
                                           self.save_percent)
        return y_BSD, sizes_N
