"""Attention over contiguous segments of a packed token sequence (images, video frames, audio windows).

Encoders attend bidirectionally inside each segment and never across.  On the GPU that is the varlen
attention kernel over the segment lengths (`ops.varlen_attention`, counterpart of the reference's
`multimodal/kernels/varlen_attention.py`); elsewhere it is torch SDPA under a block-diagonal mask that
is only built when that path runs.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ... import ops


class PackedSegments:
    def __init__(self, lens, device):
        self.lens = [int(n) for n in lens]
        self.device = device
        self._mask = None

    def mask(self) -> torch.Tensor:
        """`[1, 1, N, N]` boolean visibility."""
        if self._mask is None:
            ids = torch.repeat_interleave(torch.arange(len(self.lens)), torch.tensor(self.lens)).to(self.device)
            self._mask = (ids[:, None] == ids[None, :])[None, None]
        return self._mask

    def attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None) -> torch.Tensor:
        """`q, k, v [T, H, D]` -> `[T, H * D]`."""
        T, H, D = q.shape
        scale = D ** -0.5 if scale is None else scale
        if ops.use_native(q) and D <= 128:
            return ops.varlen_attention(q.contiguous(), k.contiguous(), v.contiguous(), self.lens, scale).reshape(T, H * D)
        o = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
                                           attn_mask=self.mask(), scale=scale)[0]
        return o.transpose(0, 1).reshape(T, H * D)
