"""LoRA hooks on the parallel linear layers (reference `python/sgl_jax/srt/lora/layers.py`).

`wrap_linear` attaches a `LoRALinear` to a `LinearBase`; its `apply(x, y)` runs after the base
GEMM and before any tensor-parallel reduction, so a row-parallel layer adds its partial
low-rank update to its partial output."""

from __future__ import annotations

import torch

from . import context_manager
from .backend.base_backend import BaseLoRABackend


class LoRALinear:
    def __init__(self, module_name: str, layer_id: int, backend: BaseLoRABackend, a_buf: torch.Tensor,
                 b_bufs: list[torch.Tensor], out_offsets: list[int]):
        self.module_name = module_name
        self.layer_id = layer_id
        self.backend = backend
        self.a_buf = a_buf                  # [slots, stack*r, in_local]
        self.b_bufs = b_bufs                # per fused member: [slots, out_local_j, r]
        self.out_offsets = out_offsets

    def apply(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        info = context_manager.current()
        if info is None or not info.has_lora:
            return y
        shape = y.shape
        y2 = y.reshape(-1, shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        return self.backend.run(x2, y2, self.a_buf, self.b_bufs, self.out_offsets, info).view(shape)


def wrap_linear(linear, lora: LoRALinear):
    linear.lora = lora
    return linear
