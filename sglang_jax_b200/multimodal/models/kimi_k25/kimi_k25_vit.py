"""Kimi-K2.5 vision tower (reference
`python/sgl_jax/srt/multimodal/models/kimi_k25/kimi_k25_vit.py`).

Patches of every frame are embedded by a strided convolution and get a learned 2-D position
table, bicubically resized to the image's patch grid and repeated over frames.  Attention is
bidirectional over all frames of one image / clip, with a 2-D rotary embedding whose interleaved
lane pairs alternate between the column and the row index.  After the last LayerNorm the frames
are averaged and each `merge_kernel_size` block of patches is concatenated; a LayerNorm + two-layer
GELU projector maps the blocks to the language model's width.

Checkpoint names: `vision_tower.patch_embed.{proj,pos_emb}`, `vision_tower.encoder.blocks.N.
{norm0,wqkv,wo,norm1,mlp.fc0,mlp.fc1}`, `vision_tower.encoder.final_layernorm`,
`mm_projector.{pre_norm,proj.0,proj.2}`."""

from __future__ import annotations

from typing import Iterable

import torch
import torch.nn.functional as F
from torch import nn

from .... import ops
from ..segments import PackedSegments


def _lin(x, lin):
    return ops.linear(x.reshape(-1, x.shape[-1]), lin.weight, lin.bias).view(*x.shape[:-1], -1)


def rope_2d(h: int, w: int, head_dim: int, theta: float = 10000.0, device=None):
    """cos/sin `[h*w, head_dim/2]`: lane pair 2i rotates with the column, pair 2i+1 with the row."""
    half = head_dim // 2
    inv = 1.0 / theta ** (torch.arange(0, half, 2, dtype=torch.float32, device=device) / half)
    fw = torch.arange(w, dtype=torch.float32, device=device)[None, :, None] * inv
    fh = torch.arange(h, dtype=torch.float32, device=device)[:, None, None] * inv
    ang = torch.stack([fw.expand(h, w, -1), fh.expand(h, w, -1)], dim=-1).reshape(h * w, half)
    return ang.cos(), ang.sin()


def apply_rope_interleaved(x, cos, sin):
    """`x [T, H, D]`; rotates (even, odd) lane pairs."""
    xf = x.float()
    a, b = xf[..., 0::2], xf[..., 1::2]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(x.shape).to(x.dtype)


class KimiVisionBlock(nn.Module):
    def __init__(self, D, heads, inter, dtype):
        super().__init__()
        self.heads = heads
        self.norm0, self.norm1 = nn.LayerNorm(D, eps=1e-6, dtype=dtype), nn.LayerNorm(D, eps=1e-6, dtype=dtype)
        self.wqkv, self.wo = nn.Linear(D, 3 * D, dtype=dtype), nn.Linear(D, D, dtype=dtype)
        self.mlp = nn.Module()
        self.mlp.fc0, self.mlp.fc1 = nn.Linear(D, inter, dtype=dtype), nn.Linear(inter, D, dtype=dtype)

    def forward(self, x, cos, sin, mask):
        T, D = x.shape
        q, k, v = _lin(self.norm0(x), self.wqkv).view(T, 3, self.heads, -1).unbind(1)
        q, k = apply_rope_interleaved(q, cos, sin), apply_rope_interleaved(k, cos, sin)
        x = x + _lin(mask.attend(q, k, v), self.wo)
        return x + _lin(F.gelu(_lin(self.norm1(x), self.mlp.fc0), approximate="tanh"), self.mlp.fc1)


class KimiK25VisionModel(nn.Module):
    """`config`: patch_size, in_channels, vt_hidden_size, vt_num_attention_heads, vt_intermediate_size,
    vt_num_hidden_layers, init_pos_emb_height / width / time, merge_kernel_size, text_hidden_size."""

    def __init__(self, config, dtype=torch.bfloat16):
        super().__init__()
        c = config
        self.config = c
        D = c.vt_hidden_size
        self.heads = c.vt_num_attention_heads
        self.merge = tuple(c.merge_kernel_size)
        self.unit = self.merge[0] * self.merge[1]
        vt = nn.Module()
        vt.patch_embed = nn.Module()
        vt.patch_embed.proj = nn.Conv2d(getattr(c, "in_channels", 3), D, c.patch_size, c.patch_size, dtype=dtype)
        vt.patch_embed.pos_emb = nn.Module()
        vt.patch_embed.pos_emb.weight = nn.Parameter(torch.zeros(c.init_pos_emb_height, c.init_pos_emb_width, D, dtype=dtype))
        vt.encoder = nn.Module()
        vt.encoder.blocks = nn.ModuleList([KimiVisionBlock(D, self.heads, c.vt_intermediate_size, dtype)
                                           for _ in range(c.vt_num_hidden_layers)])
        vt.encoder.final_layernorm = nn.LayerNorm(D, eps=1e-6, dtype=dtype)
        self.vision_tower = vt
        pj = nn.Module()
        pj.pre_norm = nn.LayerNorm(D, eps=1e-5, dtype=dtype)
        pj.proj = nn.ModuleList([nn.Linear(D * self.unit, D * self.unit, dtype=dtype), nn.GELU(),
                                 nn.Linear(D * self.unit, c.text_hidden_size, dtype=dtype)])
        self.mm_projector = pj
        self.max_frames = getattr(c, "init_pos_emb_time", 4)
        for p in self.parameters():
            p.requires_grad_(False)

    def _abs_pos(self, t, h, w):
        wt = self.vision_tower.patch_embed.pos_emb.weight
        if (h, w) != tuple(wt.shape[:2]):
            wt = F.interpolate(wt.float().permute(2, 0, 1)[None], size=(h, w), mode="bicubic",
                               align_corners=False)[0].permute(1, 2, 0).to(wt.dtype)
        return wt.reshape(h * w, -1).repeat(t, 1)

    @torch.inference_mode()
    def forward(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        """`pixel_values [sum(t*h*w), C, patch, patch]` (frame-major raster order per item), `grid_thw [n, 3]`
        -> `[sum(h*w / merge), text_hidden_size]`."""
        vt = self.vision_tower
        grids = [tuple(int(v) for v in g) for g in torch.as_tensor(grid_thw).view(-1, 3).tolist()]
        w = vt.patch_embed.proj
        x = ops.linear(pixel_values.to(w.weight.dtype).flatten(1), w.weight.flatten(1), w.bias)
        hd = x.shape[-1] // self.heads
        pos, cos, sin, ids = [], [], [], []
        for i, (t, h, wd) in enumerate(grids):
            if t > self.max_frames:
                raise ValueError(f"{t} frames exceed the position table's {self.max_frames}")
            pos.append(self._abs_pos(t, h, wd))
            c, s = rope_2d(h, wd, hd, device=x.device)
            cos.append(c.repeat(t, 1))
            sin.append(s.repeat(t, 1))
            ids.append(t * h * wd)
        x = x + torch.cat(pos).to(x.dtype)
        cos, sin = torch.cat(cos), torch.cat(sin)
        mask = PackedSegments(ids, x.device)                       # one attention segment per item
        for blk in vt.encoder.blocks:
            x = blk(x, cos, sin, mask)
        x = vt.encoder.final_layernorm(x)
        mh, mw = self.merge
        out, off = [], 0
        for t, h, wd in grids:
            item = x[off:off + t * h * wd].view(t, h // mh, mh, wd // mw, mw, -1).mean(0)     # frames pooled
            out.append(item.permute(0, 2, 1, 3, 4).reshape((h // mh) * (wd // mw), mh * mw, -1))
            off += t * h * wd
        y = self.mm_projector.pre_norm(torch.cat(out)).flatten(1)
        pj = self.mm_projector.proj
        return _lin(F.gelu(_lin(y, pj[0])), pj[2])

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            if name in params:
                params[name].data.copy_(w.to(params[name].dtype).reshape(params[name].shape))
                loaded.add(name)
        return loaded


EntryClass = [KimiK25VisionModel]
