"""`MoE`: router + MoMoE + aux-loss-free bias update, same interface as the reference wrapper
(momoe/sample_moe.py:16-68 there)."""
import torch
import torch.nn as nn

from . import ops
from .momoe import MoMoE
from .topk_router import TopKRouter


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

    def forward(self, x_BSD):
        x_BSD, mask_NM, s_NM = self.router(x_BSD, self.biases_N)
        y_BSD, sizes_N = self.momoe(x_BSD, mask_NM, s_NM)
        # DeepSeek-style auxiliary-loss-free balancing: push the bias of under-loaded experts up
        B, S, _ = x_BSD.shape
        c_avg = B * S * (self.K - self.Ks) / (self.N - self.Ks)
        with torch.no_grad():
            ops.bias_update_(self.biases_N.data, sizes_N, self.Ks, c_avg, self.bias_update_rate)
        return y_BSD
