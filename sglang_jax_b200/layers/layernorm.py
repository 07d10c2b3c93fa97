"""RMSNorm layers (reference `python/sgl_jax/srt/layers/layernorm.py:30-253`): fp32
statistics, optional fused residual add, Gemma's `(1 + w)` variant."""

from __future__ import annotations

import torch
from torch import nn

from .. import ops


class RMSNorm(nn.Module):
    gemma = False

    def __init__(self, hidden_size: int, eps: float = 1e-6, dtype=torch.bfloat16):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype), requires_grad=False)
        self.variance_epsilon = eps

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        if residual is None:
            shape = x.shape
            return ops.rmsnorm(x.reshape(-1, shape[-1]), self.weight, self.variance_epsilon, self.gemma).view(shape)
        return ops.fused_add_rmsnorm(x, residual, self.weight, self.variance_epsilon, self.gemma)

    def weight_loader(self, param, w, shard_id=None):
        param.data.copy_(w)


class GemmaRMSNorm(RMSNorm):
    gemma = True

    def __init__(self, hidden_size, eps=1e-6, dtype=torch.bfloat16):
        super().__init__(hidden_size, eps, dtype)
        self.weight.data.zero_()


class GroupRMSNorm(nn.Module):
    """RMSNorm applied independently to `num_groups` contiguous lane groups
    (reference `layers/attention/fla/group_rmsnorm.py`)."""

    def __init__(self, hidden_size, num_groups, eps=1e-6, dtype=torch.bfloat16):
        super().__init__()
        self.num_groups = num_groups
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        shape = x.shape
        g = x.reshape(-1, self.num_groups, shape[-1] // self.num_groups).float()
        y = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + self.eps)
        return (y.reshape(shape) * self.weight.float()).to(x.dtype)


class GatedRMSNorm(nn.Module):
    """`rmsnorm(x) * w * silu(gate)` used by gated-delta-net layers
    (reference `layers/attention/fla/gated_rmsnorm.py`)."""

    def __init__(self, hidden_size, eps=1e-6, dtype=torch.bfloat16):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype), requires_grad=False)
        self.eps = eps

    def weight_loader(self, param, w, shard_id=None):
        param.data.copy_(w)

    def forward(self, x, gate):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()
        return (y * torch.nn.functional.silu(gate.float())).to(x.dtype)
