"""Returns the routed expert ids per token and layer to the client (`return_routed_experts`, used
by RL pipelines; reference `python/sgl_jax/srt/layers/routed_experts_capturer.py`)."""

from __future__ import annotations

import torch


class RoutedExpertsCapturer:
    def __init__(self, num_layers: int, top_k: int, max_tokens: int, device):
        self.buf = torch.zeros((num_layers, max_tokens, top_k), dtype=torch.int32, device=device)
        self.num_tokens = 0
        self.enabled = False

    def begin(self, num_tokens: int):
        self.num_tokens = num_tokens
        self.enabled = True

    def capture(self, layer_id: int, topk_ids: torch.Tensor):
        if self.enabled:
            self.buf[layer_id, : topk_ids.shape[0]] = topk_ids

    def end(self) -> torch.Tensor:
        """`[tokens, layers, top_k]` on the host."""
        self.enabled = False
        return self.buf[:, : self.num_tokens].permute(1, 0, 2).cpu()
