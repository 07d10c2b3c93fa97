"""The Wan video VAE: causal 3-D convolutional encoder and decoder with a feature cache.

Reference: `python/sgl_jax/srt/multimodal/models/wan/vaes/wanvae.py` (`Encoder3d` :891, `Decoder3d` :772,
`AutoencoderKLWan` :1021: encode in chunks of 1 + 4k frames, decode latent frame by latent frame, every causal
convolution keeping the last two input frames of the previous chunk).

A video of `1 + 4k` frames maps to `1 + k` latent frames (8x smaller in space): the first frame is an image
(no temporal mixing in the resampling layers), later frames come in groups of four.  Time is processed in chunks;
every causal convolution remembers the tail of its previous input (`FeatureCache`), so memory is bounded by the chunk
and the output of a clip's prefix does not depend on what follows.  Weight names follow the diffusers `AutoencoderKLWan` checkpoint layout.
"""

from __future__ import annotations

from typing import Iterable

import torch
import torch.nn.functional as F
from torch import nn

CACHE_T = 2


class FeatureCache:
    """The per-layer tails of one encode / decode pass: layers take the next slot in call order."""

    def __init__(self):
        self.slots: list = []
        self.i = 0

    def rewind(self):
        self.i = 0

    def take(self):
        if self.i == len(self.slots):
            self.slots.append(None)
        self.i += 1
        return self.i - 1


class CausalConv3d(nn.Conv3d):
    """Pads only the past along time; with a cached tail of the previous chunk the padding shrinks accordingly."""

    def __init__(self, cin, cout, kernel_size, stride=1, padding=0):
        super().__init__(cin, cout, kernel_size, stride=stride, padding=0)
        p = (padding,) * 3 if isinstance(padding, int) else tuple(padding)
        self._pad = (p[2], p[2], p[1], p[1], 2 * p[0], 0)

    def forward(self, x, tail=None):
        pad = list(self._pad)
        if tail is not None and pad[4] > 0:
            x = torch.cat([tail.to(x.device), x], dim=2)
            pad[4] -= tail.shape[2]
        return super().forward(F.pad(x, pad))


def _cached_conv(conv: CausalConv3d, x, cache: FeatureCache | None):
    """Run `conv` on a chunk, feeding it the remembered tail and remembering this chunk's."""
    if cache is None:
        return conv(x)
    i = cache.take()
    prev = cache.slots[i]
    tail = x[:, :, -CACHE_T:].clone()
    if tail.shape[2] < CACHE_T and prev is not None:
        tail = torch.cat([prev[:, :, -1:].to(x.device), tail], dim=2)
    out = conv(x, prev)
    cache.slots[i] = tail
    return out


class RMSNorm(nn.Module):
    """L2 normalisation over channels times sqrt(C) and a learned gain (`gamma [C, 1, 1(, 1)]`)."""

    def __init__(self, dim, images=True):
        super().__init__()
        self.scale = dim ** 0.5
        self.gamma = nn.Parameter(torch.ones((dim, 1, 1) if images else (dim, 1, 1, 1)))

    def forward(self, x):
        return F.normalize(x.float(), dim=1).to(x.dtype) * self.scale * self.gamma


class ResidualBlock(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.norm1, self.conv1 = RMSNorm(cin, images=False), CausalConv3d(cin, cout, 3, padding=1)
        self.norm2, self.conv2 = RMSNorm(cout, images=False), CausalConv3d(cout, cout, 3, padding=1)
        self.conv_shortcut = CausalConv3d(cin, cout, 1) if cin != cout else nn.Identity()

    def forward(self, x, cache=None):
        h = self.conv_shortcut(x)
        x = _cached_conv(self.conv1, F.silu(self.norm1(x)), cache)
        x = _cached_conv(self.conv2, F.silu(self.norm2(x)), cache)
        return x + h


class AttentionBlock(nn.Module):
    """Single-head self-attention over the pixels of each frame."""

    def __init__(self, dim):
        super().__init__()
        self.norm = RMSNorm(dim)
        self.to_qkv = nn.Conv2d(dim, dim * 3, 1)
        self.proj = nn.Conv2d(dim, dim, 1)

    def forward(self, x):
        b, c, t, h, w = x.shape
        y = x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w)
        q, k, v = self.to_qkv(self.norm(y)).reshape(b * t, 1, 3 * c, h * w).transpose(2, 3).chunk(3, dim=-1)
        o = F.scaled_dot_product_attention(q, k, v).squeeze(1).transpose(1, 2).reshape(b * t, c, h, w)
        return x + self.proj(o).reshape(b, t, c, h, w).permute(0, 2, 1, 3, 4)


class Resample(nn.Module):
    """Spatial 2x up / down sampling per frame, optionally with temporal 2x through a causal convolution.  The very
    first chunk (the image frame) skips the temporal step: it neither doubles nor merges."""

    def __init__(self, dim, mode: str):
        super().__init__()
        self.mode = mode
        if mode.startswith("upsample"):
            self.resample = nn.Sequential(nn.Upsample(scale_factor=(2.0, 2.0), mode="nearest-exact"),
                                          nn.Conv2d(dim, dim // 2, 3, padding=1))
            if mode == "upsample3d":
                self.time_conv = CausalConv3d(dim, dim * 2, (3, 1, 1), padding=(1, 0, 0))
        else:
            self.resample = nn.Sequential(nn.ZeroPad2d((0, 1, 0, 1)), nn.Conv2d(dim, dim, 3, stride=(2, 2)))
            if mode == "downsample3d":
                self.time_conv = CausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0))

    def forward(self, x, cache: FeatureCache | None = None):
        b, c, t, h, w = x.shape
        if self.mode == "upsample3d" and cache is not None:
            i = cache.take()
            if cache.slots[i] is None:
                cache.slots[i] = "first"                     # the image frame: no temporal doubling
            else:
                prev = cache.slots[i]
                tail = x[:, :, -CACHE_T:].clone()
                if tail.shape[2] < CACHE_T:
                    head = torch.zeros_like(tail) if isinstance(prev, str) else prev[:, :, -1:].to(x.device)
                    tail = torch.cat([head, tail], dim=2)
                x = self.time_conv(x) if isinstance(prev, str) else self.time_conv(x, prev)
                cache.slots[i] = tail
                x = x.reshape(b, 2, c, t, h, w)
                x = torch.stack((x[:, 0], x[:, 1]), dim=3).reshape(b, c, t * 2, h, w)
        t = x.shape[2]
        y = x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w)
        y = self.resample[1](self.resample[0](y.float()).to(y.dtype)) if self.mode.startswith("upsample") else self.resample(y)
        x = y.reshape(b, t, *y.shape[1:]).permute(0, 2, 1, 3, 4)
        if self.mode == "downsample3d" and cache is not None:
            i = cache.take()
            if cache.slots[i] is None:
                cache.slots[i] = x.clone()                   # the image frame passes through
            else:
                last = x[:, :, -1:].clone()
                x = self.time_conv(torch.cat([cache.slots[i][:, :, -1:].to(x.device), x], dim=2))
                cache.slots[i] = last
        return x


class MidBlock(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.resnets = nn.ModuleList([ResidualBlock(dim, dim), ResidualBlock(dim, dim)])
        self.attentions = nn.ModuleList([AttentionBlock(dim)])

    def forward(self, x, cache=None):
        return self.resnets[1](self.attentions[0](self.resnets[0](x, cache)), cache)


class Encoder3d(nn.Module):
    def __init__(self, dim=96, z_dim=32, dim_mult=(1, 2, 4, 4), num_res_blocks=2, temporal_downsample=(False, True, True),
                 in_channels=3):
        super().__init__()
        dims = [dim * m for m in (1,) + tuple(dim_mult)]
        self.conv_in = CausalConv3d(in_channels, dims[0], 3, padding=1)
        blocks = []
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            for _ in range(num_res_blocks):
                blocks.append(ResidualBlock(cin, cout))
                cin = cout
            if i != len(dim_mult) - 1:
                blocks.append(Resample(cout, "downsample3d" if temporal_downsample[i] else "downsample2d"))
        self.down_blocks = nn.ModuleList(blocks)
        self.mid_block = MidBlock(dims[-1])
        self.norm_out = RMSNorm(dims[-1], images=False)
        self.conv_out = CausalConv3d(dims[-1], z_dim, 3, padding=1)

    def forward(self, x, cache=None):
        x = _cached_conv(self.conv_in, x, cache)
        for blk in self.down_blocks:
            x = blk(x, cache)
        x = self.mid_block(x, cache)
        return _cached_conv(self.conv_out, F.silu(self.norm_out(x)), cache)


class UpBlock(nn.Module):
    def __init__(self, cin, cout, num_res_blocks, mode: str | None):
        super().__init__()
        res = []
        for _ in range(num_res_blocks + 1):
            res.append(ResidualBlock(cin, cout))
            cin = cout
        self.resnets = nn.ModuleList(res)
        self.upsamplers = nn.ModuleList([Resample(cout, mode)]) if mode else None

    def forward(self, x, cache=None):
        for r in self.resnets:
            x = r(x, cache)
        if self.upsamplers is not None:
            x = self.upsamplers[0](x, cache)
        return x


class Decoder3d(nn.Module):
    def __init__(self, dim=96, z_dim=16, dim_mult=(1, 2, 4, 4), num_res_blocks=2, temporal_upsample=(True, True, False),
                 out_channels=3):
        super().__init__()
        dims = [dim * m for m in (dim_mult[-1],) + tuple(dim_mult[::-1])]
        self.conv_in = CausalConv3d(z_dim, dims[0], 3, padding=1)
        self.mid_block = MidBlock(dims[0])
        ups = []
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            if i > 0:
                cin = cin // 2                                # the previous level's upsampler halved the channels
            mode = None
            if i != len(dim_mult) - 1:
                mode = "upsample3d" if temporal_upsample[i] else "upsample2d"
            ups.append(UpBlock(cin, cout, num_res_blocks, mode))
        self.up_blocks = nn.ModuleList(ups)
        self.norm_out = RMSNorm(dims[-1], images=False)
        self.conv_out = CausalConv3d(dims[-1], out_channels, 3, padding=1)

    def forward(self, x, cache=None):
        x = _cached_conv(self.conv_in, x, cache)
        x = self.mid_block(x, cache)
        for blk in self.up_blocks:
            x = blk(x, cache)
        return _cached_conv(self.conv_out, F.silu(self.norm_out(x)), cache)


class WanVAE(nn.Module):
    """`config`: base_dim, z_dim, dim_mult, num_res_blocks, temporal_downsample, latents_mean / latents_std (per
    latent channel; identity when absent)."""

    def __init__(self, config, dtype=torch.float32, quant_config=None):
        super().__init__()
        c = config
        self.config = c
        z = c.z_dim
        # (released checkpoints spell the field `temperal_downsample`)
        td = tuple(getattr(c, "temporal_downsample", None) or getattr(c, "temperal_downsample", None) or (False, True, True))
        kw = dict(dim=c.base_dim, dim_mult=tuple(c.dim_mult), num_res_blocks=getattr(c, "num_res_blocks", 2))
        self.encoder = Encoder3d(z_dim=2 * z, temporal_downsample=td, in_channels=getattr(c, "in_channels", 3), **kw)
        self.quant_conv = CausalConv3d(2 * z, 2 * z, 1)
        self.post_quant_conv = CausalConv3d(z, z, 1)
        self.decoder = Decoder3d(z_dim=z, temporal_upsample=td[::-1], out_channels=getattr(c, "out_channels", 3), **kw)
        mean = torch.tensor(getattr(c, "latents_mean", None) or [0.0] * z).view(1, z, 1, 1, 1)
        std = torch.tensor(getattr(c, "latents_std", None) or [1.0] * z).view(1, z, 1, 1, 1)
        self.register_buffer("latents_mean", mean, persistent=False)
        self.register_buffer("latents_std", std, persistent=False)
        self.to(dtype)

    @torch.inference_mode()
    def encode(self, video: torch.Tensor, sample: bool = False, generator=None) -> torch.Tensor:
        """`video [B, C, 1 + 4k, H, W]` in [-1, 1] -> normalised latents `[B, z, 1 + k, H / 8, W / 8]` (the mean of
        the posterior, or a sample of it)."""
        x = video.to(self.quant_conv.weight.dtype)
        cache = FeatureCache()
        t = x.shape[2]
        outs = []
        for i in range(1 + max(t - 1, 0) // 4):
            cache.rewind()
            chunk = x[:, :, :1] if i == 0 else x[:, :, 1 + 4 * (i - 1):1 + 4 * i]
            outs.append(self.encoder(chunk, cache))
        mu, logvar = self.quant_conv(torch.cat(outs, dim=2)).chunk(2, dim=1)
        if sample:
            mu = mu + torch.exp(0.5 * logvar.clamp(-30, 20)) * torch.randn(mu.shape, generator=generator, dtype=mu.dtype,
                                                                          device=mu.device)
        return (mu - self.latents_mean.to(mu)) / self.latents_std.to(mu)

    @torch.inference_mode()
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        """Normalised latents `[B, z, 1 + k, h, w]` -> video `[B, C, 1 + 4k, 8h, 8w]` in [-1, 1]."""
        z = z.to(self.post_quant_conv.weight.dtype) * self.latents_std.to(z.device) + self.latents_mean.to(z.device)
        x = self.post_quant_conv(z.to(self.post_quant_conv.weight.dtype))
        cache = FeatureCache()
        outs = []
        for i in range(x.shape[2]):
            cache.rewind()
            outs.append(self.decoder(x[:, :, i:i + 1], cache))
        return torch.cat(outs, dim=2).clamp(-1, 1)

    forward = decode

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            if name in params and tuple(params[name].shape) == tuple(w.shape):
                params[name].data.copy_(w.to(params[name].dtype))
                loaded.add(name)
        return loaded
