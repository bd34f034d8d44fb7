"""B200-native MoMoE layer: drop-in `MoMoE`, `MoE`, `TopKRouter` running on libmomoe_b200.so."""
from .momoe import MoMoE
from .sample_moe import MoE
from .topk_router import TopKRouter

__all__ = ["MoMoE", "MoE", "TopKRouter"]
