"""Routed expert ids per token and layer, returned to the client with `return_routed_experts`
(RL pipelines replay the router's choices; reference
`python/sgl_jax/srt/layers/routed_experts_capturer.py`: a host ring plus per-request slicing).

Device side: one static `[layers, max_tokens, top_k]` int32 buffer that every MoE layer writes its
(logical) top-k ids into, so the copies are part of captured CUDA graphs too.  After a forward the
first `num_tokens` rows are copied to pinned host memory without blocking the stream; the scheduler
slices the host copy per request once the step's results are resolved."""

from __future__ import annotations

import numpy as np
import torch


class RoutedExpertsCapturer:
    def __init__(self, num_layers: int, top_k: int, max_tokens: int, device):
        self.num_layers, self.top_k, self.max_tokens = num_layers, top_k, max_tokens
        self.device = torch.device(device)
        self.buf = torch.zeros((num_layers, max_tokens, top_k), dtype=torch.int32, device=self.device)

    @classmethod
    def attach(cls, model, max_tokens: int, device, top_k: int = 8) -> "RoutedExpertsCapturer | None":
        """Create a capturer for `model` and hook it into every routed-expert layer (None for dense models)."""
        from .moe import FusedMoE
        moes = [m for m in model.modules() if isinstance(m, FusedMoE)]
        if not moes:
            return None
        cap = cls(max(m.layer_id for m in moes) + 1, top_k, max_tokens, device)
        for m in moes:
            m.routed_experts_capturer = cap
        return cap

    def capture(self, layer_id: int, topk_ids: torch.Tensor):
        T, k = topk_ids.shape
        if T <= self.max_tokens and k <= self.top_k:
            self.buf[layer_id, :T, :k] = topk_ids

    def snapshot(self, num_tokens: int):
        """Start the device -> pinned host copy of the last forward's ids: `(host tensor [layers, tokens, top_k],
        event | None)`; the tensor is valid once the event has completed."""
        n = min(num_tokens, self.max_tokens)
        if self.device.type != "cuda":
            return self.buf[:, :n].clone(), None
        host = torch.empty((self.num_layers, n, self.top_k), dtype=torch.int32, pin_memory=True)
        host.copy_(self.buf[:, :n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return host, ev

    @staticmethod
    def per_request(host: torch.Tensor, event, row_spans: list[tuple[int, int]]) -> list[np.ndarray]:
        """Slice a snapshot into `[tokens_of_request, layers, top_k]` arrays for the row spans `(first, count)`."""
        if event is not None:
            event.synchronize()
        arr = host.numpy().transpose(1, 0, 2)
        return [arr[a:a + n].copy() for a, n in row_spans]
