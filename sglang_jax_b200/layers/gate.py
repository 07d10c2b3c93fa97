"""Router: gate logits and top-k selection (reference `python/sgl_jax/srt/layers/gate.py`:
`GateLogit` :59 — fp32 `hidden . Wg` with softmax / sigmoid / tanh scoring; `TopK` :109 — plain,
biased, grouped and biased-grouped selection, renormalisation, `routed_scaling_factor`)."""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops


class GateLogit(nn.Module):
    """Replicated router projection.  Logits are computed in fp32 (the top-k choice is sensitive to
    rounding); the optional selection bias (`e_score_correction_bias`) lives here too."""

    def __init__(self, hidden_size: int, num_experts: int, dtype=torch.bfloat16, use_bias: bool = False,
                 score_func: str = "softmax", correction_bias: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, hidden_size, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(num_experts, dtype=dtype), requires_grad=False) if use_bias else None
        self.e_score_correction_bias = nn.Parameter(torch.zeros(num_experts, dtype=torch.float32),
                                                    requires_grad=False) if correction_bias else None
        self.score_func = score_func

    def weight_loader(self, param, w, shard_id=None):
        param.data.copy_(w)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x.float(), self.weight.float(), self.bias.float() if self.bias is not None else None)


class TopK(nn.Module):
    def __init__(self, top_k: int, renormalize: bool = True, num_expert_group: int = 0, topk_group: int = 0,
                 routed_scaling_factor: float = 1.0, scoring_func: str = "softmax"):
        super().__init__()
        self.top_k = top_k
        self.renormalize = renormalize
        self.num_expert_group = num_expert_group or 0
        self.topk_group = topk_group or 0
        self.routed_scaling_factor = routed_scaling_factor or 1.0
        self.scoring_func = scoring_func
        self.expert_location = None     # eplb.ExpertLocation: logical -> physical ids

    def forward(self, router_logits: torch.Tensor, correction_bias: torch.Tensor | None = None):
        w, ids = ops.topk_route(router_logits, self.top_k, self.scoring_func, self.renormalize, correction_bias,
                                self.num_expert_group, self.topk_group, self.routed_scaling_factor)
        if self.expert_location is not None:
            ids = self.expert_location.logical_to_physical(ids)
        return w, ids
