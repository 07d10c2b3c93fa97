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


class _Resnet2d(nn.Module):
    def __init__(self, cin, cout, groups):
        super().__init__()
        self.norm1, self.conv1 = nn.GroupNorm(groups, cin, eps=1e-6), nn.Conv2d(cin, cout, 3, padding=1)
        self.norm2, self.conv2 = nn.GroupNorm(groups, cout, eps=1e-6), nn.Conv2d(cout, cout, 3, padding=1)
        self.conv_shortcut = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.conv2(F.silu(self.norm2(self.conv1(F.silu(self.norm1(x))))))
        return (x if self.conv_shortcut is None else self.conv_shortcut(x)) + h


class _MidAttention(nn.Module):
    """Single-head self-attention over the spatial positions of the coarsest feature map."""

    def __init__(self, c, groups):
        super().__init__()
        self.group_norm = nn.GroupNorm(groups, c, eps=1e-6)
        self.to_q, self.to_k, self.to_v = nn.Linear(c, c), nn.Linear(c, c), nn.Linear(c, c)
        self.to_out = nn.ModuleList([nn.Linear(c, c)])

    def forward(self, x):
        B, C, H, W = x.shape
        h = self.group_norm(x).flatten(2).transpose(1, 2)
        a = F.scaled_dot_product_attention(self.to_q(h)[:, None], self.to_k(h)[:, None], self.to_v(h)[:, None])[:, 0]
        return x + self.to_out[0](a).transpose(1, 2).reshape(B, C, H, W)


class _Mid(nn.Module):
    def __init__(self, c, groups, attention=True):
        super().__init__()
        self.resnets = nn.ModuleList([_Resnet2d(c, c, groups), _Resnet2d(c, c, groups)])
        self.attentions = nn.ModuleList([_MidAttention(c, groups)]) if attention else None

    def forward(self, x):
        x = self.resnets[0](x)
        if self.attentions is not None:
            x = self.attentions[0](x)
        return self.resnets[1](x)


class _Sampler(nn.Module):
    def __init__(self, c, down: bool):
        super().__init__()
        self.down = down
        self.conv = nn.Conv2d(c, c, 3, stride=2 if down else 1, padding=0 if down else 1)

    def forward(self, x):
        if self.down:
            return self.conv(F.pad(x, (0, 1, 0, 1)))
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))


class _Level(nn.Module):
    def __init__(self, cin, cout, n, groups, sampler: str | None):
        super().__init__()
        self.resnets = nn.ModuleList([_Resnet2d(cin if i == 0 else cout, cout, groups) for i in range(n)])
        if sampler == "down":
            self.downsamplers = nn.ModuleList([_Sampler(cout, True)])
        elif sampler == "up":
            self.upsamplers = nn.ModuleList([_Sampler(cout, False)])
        self._s = sampler

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        if self._s == "down":
            x = self.downsamplers[0](x)
        elif self._s == "up":
            x = self.upsamplers[0](x)
        return x


class _Encoder2d(nn.Module):
    def __init__(self, cin, chans, layers, groups, latent, attention):
        super().__init__()
        self.conv_in = nn.Conv2d(cin, chans[0], 3, padding=1)
        self.down_blocks = nn.ModuleList([
            _Level(chans[max(i - 1, 0)], c, layers, groups, "down" if i < len(chans) - 1 else None)
            for i, c in enumerate(chans)])
        self.mid_block = _Mid(chans[-1], groups, attention)
        self.conv_norm_out = nn.GroupNorm(groups, chans[-1], eps=1e-6)
        self.conv_out = nn.Conv2d(chans[-1], 2 * latent, 3, padding=1)

    def forward(self, x):
        x = self.conv_in(x)
        for b in self.down_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(self.mid_block(x))))


class _Decoder2d(nn.Module):
    def __init__(self, cout, chans, layers, groups, latent, attention):
        super().__init__()
        rev = list(reversed(chans))
        self.conv_in = nn.Conv2d(latent, rev[0], 3, padding=1)
        self.mid_block = _Mid(rev[0], groups, attention)
        self.up_blocks = nn.ModuleList([
            _Level(rev[max(i - 1, 0)], c, layers + 1, groups, "up" if i < len(rev) - 1 else None)
            for i, c in enumerate(rev)])
        self.conv_norm_out = nn.GroupNorm(groups, rev[-1], eps=1e-6)
        self.conv_out = nn.Conv2d(rev[-1], cout, 3, padding=1)

    def forward(self, z):
        x = self.mid_block(self.conv_in(z))
        for b in self.up_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


class AutoencoderKL(nn.Module):
    """Image VAE of the latent-diffusion family (Flux, SD): residual conv levels with a
    single-head attention block at the coarsest resolution; the encoder halves and the decoder
    doubles the resolution between levels.  Parameter names follow the published checkpoints
    (`encoder.down_blocks.N.resnets.M.*`, `decoder.up_blocks.N.upsamplers.0.conv`, `mid_block.attentions.0.to_q`, ...).
    `config`: in_channels, out_channels, latent_channels, block_out_channels, layers_per_block,
    norm_num_groups, scaling_factor, shift_factor, use_quant_conv / use_post_quant_conv.
    Reference: `python/sgl_jax/srt/multimodal/models/vaes/autoencoder.py`, `vaes/common.py`."""

    def __init__(self, config, dtype=torch.float32, quant_config=None):
        super().__init__()
        c = config
        self.config = c
        latent = getattr(c, "latent_channels", None) or getattr(c, "z_dim", 16)
        chans = list(getattr(c, "block_out_channels", None) or
                     [c.base_dim * m for m in reversed(c.dim_mult)])
        layers = getattr(c, "layers_per_block", 2)
        groups = getattr(c, "norm_num_groups", None) or min(8, min(chans))
        attn = bool(getattr(c, "mid_block_add_attention", True))
        self.latent_channels = latent
        self.encoder = _Encoder2d(getattr(c, "in_channels", 3), chans, layers, groups, latent, attn)
        self.decoder = _Decoder2d(getattr(c, "out_channels", 3), chans, layers, groups, latent, attn)
        self.quant_conv = nn.Conv2d(2 * latent, 2 * latent, 1) if getattr(c, "use_quant_conv", False) else None
        self.post_quant_conv = nn.Conv2d(latent, latent, 1) if getattr(c, "use_post_quant_conv", False) else None
        self.scaling_factor = float(getattr(c, "scaling_factor", 1.0) or 1.0)
        self.shift_factor = float(getattr(c, "shift_factor", 0.0) or 0.0)
        self.spatial_factor = 2 ** (len(chans) - 1)
        for p in self.parameters():
            p.requires_grad_(False)
        self.to(dtype)

    @torch.inference_mode()
    def encode(self, pixels: torch.Tensor, sample: bool = False, generator=None) -> torch.Tensor:
        """`pixels [B, 3, H, W]` in [-1, 1] -> scaled latents `[B, latent, H/f, W/f]` (the posterior mean,
        or a sample of it)."""
        h = self.encoder(pixels.to(self.encoder.conv_in.weight.dtype))
        if self.quant_conv is not None:
            h = self.quant_conv(h)
        mean, logvar = h.chunk(2, dim=1)
        if sample:
            mean = mean + torch.exp(0.5 * logvar.clamp(-30, 20)) * torch.randn(mean.shape, generator=generator).to(mean)
        return (mean - self.shift_factor) * self.scaling_factor

    @torch.inference_mode()
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        """`z [B, latent, H, W]` or `[B, latent, T, H, W]` (frames decoded independently) -> pixels in [-1, 1]."""
        five = z.dim() == 5
        if five:
            B, C, T, H, W = z.shape
            z = z.permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W)
        z = z.to(self.decoder.conv_in.weight.dtype) / self.scaling_factor + self.shift_factor
        if self.post_quant_conv is not None:
            z = self.post_quant_conv(z)
        x = self.decoder(z).clamp(-1, 1)
        if five:
            x = x.view(B, T, *x.shape[1:]).permute(0, 2, 1, 3, 4)
        return x

    forward = decode

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            # older checkpoints name the attention projections query/key/value/proj_attn
            n = (name.replace(".query.", ".to_q.").replace(".key.", ".to_k.").replace(".value.", ".to_v.")
                 .replace(".proj_attn.", ".to_out.0."))
            if n in params:
                params[n].data.copy_(w.to(params[n].dtype).reshape(params[n].shape))
                loaded.add(n)
        return loaded


EntryClass = [AutoencoderKLWan, AutoencoderKL]
