"""Qwen3-Omni / Qwen3-VL vision encoder (reference
`python/sgl_jax/srt/multimodal/models/qwen3_omni_moe/vision_encoder.py`).

Patches (`temporal_patch_size x patch x patch` voxels, already ordered in `merge x merge` groups)
are embedded by one linear map; a learned `sqrt(num_position_embeddings)`-sided position table is
bilinearly interpolated to each image's grid; attention is full within a frame with 2-D rotary
positions (row lanes, column lanes).  The final merger concatenates each `merge x merge` group
into one token; `deepstack_visual_indexes` name intermediate layers whose merged features are
handed to the first layers of the language model."""

from __future__ import annotations

from typing import Iterable

import torch
import torch.nn.functional as F
from torch import nn

from .... import ops
from ..segments import PackedSegments


def _lin(x, lin):
    return ops.linear(x.reshape(-1, x.shape[-1]), lin.weight, lin.bias).view(*x.shape[:-1], -1)


def _act(name):
    return {"gelu": F.gelu, "gelu_pytorch_tanh": lambda x: F.gelu(x, approximate="tanh"), "silu": F.silu,
            "quick_gelu": lambda x: x * torch.sigmoid(1.702 * x)}[name]


class VisionBlock(nn.Module):
    def __init__(self, c, dtype):
        super().__init__()
        D = c.hidden_size
        self.heads = c.num_heads
        self.norm1, self.norm2 = nn.LayerNorm(D, eps=1e-6, dtype=dtype), nn.LayerNorm(D, eps=1e-6, dtype=dtype)
        self.attn = nn.Module()
        self.attn.qkv, self.attn.proj = nn.Linear(D, 3 * D, dtype=dtype), nn.Linear(D, D, dtype=dtype)
        self.mlp = nn.Module()
        self.mlp.linear_fc1 = nn.Linear(D, c.intermediate_size, dtype=dtype)
        self.mlp.linear_fc2 = nn.Linear(c.intermediate_size, D, dtype=dtype)
        self.act = _act(getattr(c, "hidden_act", "gelu_pytorch_tanh"))

    def forward(self, x, cos, sin, mask):
        T, D = x.shape
        q, k, v = _lin(self.norm1(x), self.attn.qkv).view(T, 3, self.heads, -1).unbind(1)

        def rot(t):
            tf = t.float()
            h = tf.shape[-1] // 2
            return (tf * cos + torch.cat([-tf[..., h:], tf[..., :h]], -1) * sin).to(t.dtype)

        q, k = rot(q), rot(k)
        x = x + _lin(mask.attend(q, k, v), self.attn.proj)
        return x + _lin(self.act(_lin(self.norm2(x), self.mlp.linear_fc1)), self.mlp.linear_fc2)


class PatchMerger(nn.Module):
    def __init__(self, c, dtype, postshuffle_norm: bool):
        super().__init__()
        self.width = c.hidden_size * c.spatial_merge_size ** 2
        self.post = postshuffle_norm
        self.ln_q = nn.LayerNorm(self.width if postshuffle_norm else c.hidden_size, eps=1e-6, dtype=dtype)
        self.mlp = nn.ModuleList([nn.Linear(self.width, self.width, dtype=dtype), nn.GELU(),
                                  nn.Linear(self.width, c.out_hidden_size, dtype=dtype)])

    def forward(self, x):
        x = self.ln_q(x.view(-1, self.width) if self.post else x).view(-1, self.width)
        return _lin(F.gelu(_lin(x, self.mlp[0])), self.mlp[2])


class Qwen3OmniMoeVisionEncoder(nn.Module):
    def __init__(self, config, dtype=torch.bfloat16):
        super().__init__()
        c = config
        self.config = c
        self.merge = c.spatial_merge_size
        self.unit = self.merge ** 2
        D = c.hidden_size
        self.patch_dim = c.in_channels * c.temporal_patch_size * c.patch_size ** 2
        self.patch_embed = nn.Module()
        self.patch_embed.proj = nn.Conv3d(c.in_channels, D, (c.temporal_patch_size, c.patch_size, c.patch_size),
                                          (c.temporal_patch_size, c.patch_size, c.patch_size), dtype=dtype)
        self.pos_embed = nn.Embedding(c.num_position_embeddings, D, dtype=dtype)
        self.side = int(c.num_position_embeddings ** 0.5)
        self.blocks = nn.ModuleList([VisionBlock(c, dtype) for _ in range(c.depth)])
        self.merger = PatchMerger(c, dtype, False)
        self.deepstack_visual_indexes = list(getattr(c, "deepstack_visual_indexes", []) or [])
        self.merger_list = nn.ModuleList([PatchMerger(c, dtype, True) for _ in self.deepstack_visual_indexes])
        hd = D // c.num_heads
        self.register_buffer("inv_freq", 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float) / (hd // 2))),
                             persistent=False)
        for p in self.parameters():
            p.requires_grad_(False)

    def _grouped(self, t, h, w, per_patch):
        """`per_patch [h*w, ...]` in raster order -> frame-repeated, `merge x merge`-grouped order."""
        m = self.merge
        x = per_patch.view(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
        return x.repeat(t, 1)

    def _positions(self, grid):
        dev = self.pos_embed.weight.device
        embeds, angles = [], []
        for t, h, w in grid.tolist():
            hs, ws = torch.linspace(0, self.side - 1, h), torch.linspace(0, self.side - 1, w)
            hf, wf = hs.int(), ws.int()
            hc, wc = (hf + 1).clip(max=self.side - 1), (wf + 1).clip(max=self.side - 1)
            dh, dw = (hs - hf)[:, None], (ws - wf)[None, :]
            table = self.pos_embed.weight

            def at(a, b):
                return table[(a[:, None] * self.side + b[None, :]).flatten().long().to(dev)]
            wts = [((1 - dh) * (1 - dw)), ((1 - dh) * dw), (dh * (1 - dw)), (dh * dw)]
            pe = sum(at(a, b) * wt.flatten()[:, None].to(table) for (a, b), wt in
                     zip([(hf, wf), (hf, wc), (hc, wf), (hc, wc)], wts))
            embeds.append(self._grouped(t, h, w, pe))
            rc = torch.stack(torch.meshgrid(torch.arange(h), torch.arange(w), indexing="ij"), -1).view(h * w, 2)
            rc = self._grouped(t, h, w, rc.float()).to(dev)
            angles.append((rc[:, :, None] * self.inv_freq[None, None, :]).flatten(1))
        return torch.cat(embeds), torch.cat(angles)

    @torch.inference_mode()
    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor, return_deepstack: bool = False):
        """`pixel_values [sum(t*h*w), patch_dim]`, `grid_thw [n, 3]` -> `[sum(t*h*w)/merge^2, out_hidden_size]`
        (and the list of deep-stack features, one per `deepstack_visual_indexes` entry)."""
        w = self.patch_embed.proj
        x = ops.linear(pixel_values.to(w.weight.dtype), w.weight.view(w.weight.shape[0], -1), w.bias)
        pos, ang = self._positions(grid_thw)
        x = x + pos.to(x.dtype)
        ang = torch.cat([ang, ang], dim=-1)
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        frames = torch.repeat_interleave(grid_thw[:, 1] * grid_thw[:, 2], grid_thw[:, 0])
        mask = PackedSegments(frames.tolist(), x.device)          # one attention segment per frame
        deep = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, mask)
            if i in self.deepstack_visual_indexes:
                deep.append(self.merger_list[self.deepstack_visual_indexes.index(i)](x))
        out = self.merger(x)
        return (out, deep) if return_deepstack else out

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            n = name.split("visual.", 1)[-1]
            if n in params:
                params[n].data.copy_(w.to(params[n].dtype))
                loaded.add(n)
        return loaded


EntryClass = [Qwen3OmniMoeVisionEncoder]
