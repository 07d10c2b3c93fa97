"""Latent decoders (reference `multimodal/models/vaes`, `multimodal/models/wan` WanVAE): a
convolutional decoder that upsamples latents 8x spatially (and, for video, 4x in time with
causal temporal convolutions) to pixels."""

from __future__ import annotations

from typing import Iterable

import torch
import torch.nn.functional as F
from torch import nn


class CausalConv3d(nn.Conv3d):
    """3-D convolution that pads only the past along time, so frame t never sees later frames."""

    def forward(self, x):
        kt, kh, kw = self.kernel_size
        x = F.pad(x, (kw // 2, kw // 2, kh // 2, kh // 2, kt - 1, 0))
        return F.conv3d(x, self.weight, self.bias, self.stride, 0, self.dilation, self.groups)


class ResBlock3d(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.n1, self.c1 = nn.GroupNorm(min(8, cin), cin), CausalConv3d(cin, cout, 3)
        self.n2, self.c2 = nn.GroupNorm(min(8, cout), cout), CausalConv3d(cout, cout, 3)
        self.skip = CausalConv3d(cin, cout, 1) if cin != cout else nn.Identity()

    def forward(self, x):
        h = self.c1(F.silu(self.n1(x)))
        h = self.c2(F.silu(self.n2(h)))
        return self.skip(x) + h


class AutoencoderKLWan(nn.Module):
    """`config`: z_dim, base_dim, dim_mult (coarse -> fine), temporal_upsample (per level), out_channels,
    scaling_factor."""

    def __init__(self, config, dtype=torch.float32, quant_config=None):
        super().__init__()
        c = config
        self.config = c
        dims = [c.base_dim * m for m in c.dim_mult]
        self.conv_in = CausalConv3d(c.z_dim, dims[0], 3)
        blocks, ups = [], []
        for i, d in enumerate(dims):
            blocks.append(ResBlock3d(dims[i - 1] if i else dims[0], d))
            ups.append(bool(c.temporal_upsample[i]) if i < len(c.temporal_upsample) else False)
        self.blocks = nn.ModuleList(blocks)
        self.temporal_up = ups
        self.norm_out = nn.GroupNorm(min(8, dims[-1]), dims[-1])
        self.conv_out = CausalConv3d(dims[-1], c.out_channels, 3)
        self.to(dtype)

    @torch.inference_mode()
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        """`z [B, z_dim, T, H, W]` -> pixels `[B, out_channels, T', 8H, 8W]` in [-1, 1]."""
        x = self.conv_in(z.to(self.conv_in.weight.dtype) / self.config.scaling_factor)
        n = len(self.blocks)
        for i, blk in enumerate(self.blocks):
            x = blk(x)
            if i < n - 1 or n == 1:
                st = 2 if self.temporal_up[i] and x.shape[2] > 1 else 1
                x = F.interpolate(x, scale_factor=(st, 2, 2), mode="nearest")
        return torch.tanh(self.conv_out(F.silu(self.norm_out(x))))

    forward = decode

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            if name in params:
                params[name].data.copy_(w.to(params[name].dtype))
                loaded.add(name)
        return loaded


class AutoencoderKL(AutoencoderKLWan):
    """Image VAE: the same decoder on a single frame."""


EntryClass = [AutoencoderKLWan, AutoencoderKL]
