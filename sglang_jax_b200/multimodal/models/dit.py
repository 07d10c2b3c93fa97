"""Diffusion transformers: the Wan-style video DiT (self-attention over the 3-D latent patch grid
with rotary position in (t, h, w), cross-attention to the text tokens, adaLN modulation from the
timestep; reference `multimodal/models/wan`).  The Flux image DiT lives in `flux.py`.

Attention here is dense and bidirectional; projections and FFNs are `ops.linear`, i.e. the
tcgen05 GEMM on a GPU."""

from __future__ import annotations

import math
from typing import Iterable

import torch
from torch import nn

from ... import ops


def _lin(o, i, dtype, bias=True):
    m = nn.Module()
    m.weight = nn.Parameter(torch.empty(o, i, dtype=dtype), requires_grad=False)
    m.bias = nn.Parameter(torch.zeros(o, dtype=dtype), requires_grad=False) if bias else None
    return m


def _apply(m, x):
    shape = x.shape
    return ops.linear(x.reshape(-1, shape[-1]), m.weight, m.bias).view(*shape[:-1], m.weight.shape[0])


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


def rope_3d(grid: tuple[int, int, int], head_dim: int, device, theta: float = 10000.0):
    """cos/sin `[N, head_dim/2]` for a (T, H, W) grid: the head is split into three bands that
    rotate with the frame, row and column index."""
    T, H, W = grid
    d_t = head_dim // 2 - 2 * (head_dim // 6)
    d_h = d_w = head_dim // 6
    def band(n, d):
        inv = 1.0 / theta ** (torch.arange(d, dtype=torch.float32, device=device) / max(d, 1))
        return torch.arange(n, dtype=torch.float32, device=device)[:, None] * inv[None]
    ft, fh, fw = band(T, d_t), band(H, d_h), band(W, d_w)
    ang = torch.cat([ft[:, None, None, :].expand(T, H, W, d_t), fh[None, :, None, :].expand(T, H, W, d_h),
                     fw[None, None, :, :].expand(T, H, W, d_w)], dim=-1).reshape(T * H * W, -1)
    return ang.cos(), ang.sin()


def apply_rope_pairs(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """`x [B, N, H, D]`, interleaved (even, odd) pairs."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    a, b = xf[..., 0], xf[..., 1]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.stack([a * c - b * s, a * s + b * c], dim=-1).reshape(x.shape).to(x.dtype)


def _rms(x, w, eps=1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def _ln(x, eps=1e-6):
    return torch.nn.functional.layer_norm(x.float(), x.shape[-1:], eps=eps).to(x.dtype)


def _sdpa(q, k, v):
    return torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
                                                            ).transpose(1, 2)


def _self_attention(q, k, v):
    """Dense bidirectional self-attention `[B, N, H, D]`.  On the GPU (bf16, head dim up to 128) the batch is one
    packed sequence list for the varlen attention kernel (tcgen05 for head dim 128), counterpart of the reference's
    `multimodal/kernels/flash_attention.py`; elsewhere torch SDPA."""
    B, N, H, D = q.shape
    from ... import ops
    if ops.use_native(q) and q.dtype == torch.bfloat16 and D in (64, 128):
        o = ops.varlen_attention(q.reshape(B * N, H, D).contiguous(), k.reshape(B * N, H, D).contiguous(),
                                 v.reshape(B * N, H, D).contiguous(), [N] * B, D ** -0.5)
        return o.reshape(B, N, H, D)
    return _sdpa(q, k, v)


class WanBlock(nn.Module):
    def __init__(self, dim, heads, ffn, dtype):
        super().__init__()
        self.heads = heads
        for n in ("q", "k", "v", "o", "cq", "ck", "cv", "co"):
            setattr(self, n, _lin(dim, dim, dtype))
        self.norm_q = nn.Parameter(torch.ones(dim, dtype=dtype), requires_grad=False)
        self.norm_k = nn.Parameter(torch.ones(dim, dtype=dtype), requires_grad=False)
        self.norm_cq = nn.Parameter(torch.ones(dim, dtype=dtype), requires_grad=False)
        self.norm_ck = nn.Parameter(torch.ones(dim, dtype=dtype), requires_grad=False)
        self.norm3_w = nn.Parameter(torch.ones(dim, dtype=dtype), requires_grad=False)
        self.norm3_b = nn.Parameter(torch.zeros(dim, dtype=dtype), requires_grad=False)
        self.ffn_in, self.ffn_out = _lin(ffn, dim, dtype), _lin(dim, ffn, dtype)
        self.modulation = nn.Parameter(torch.zeros(1, 6, dim, dtype=dtype), requires_grad=False)

    def forward(self, x, ctx, e, cos, sin):
        B, N, D = x.shape
        H = self.heads
        m = (self.modulation.float() + e.float()).unbind(1)            # 6 x [B, D]: shift/scale/gate x2
        h = _ln(x) * (1 + m[1][:, None]) + m[0][:, None]
        h = h.to(x.dtype)
        q = _rms(_apply(self.q, h), self.norm_q).view(B, N, H, -1)
        k = _rms(_apply(self.k, h), self.norm_k).view(B, N, H, -1)
        v = _apply(self.v, h).view(B, N, H, -1)
        a = _self_attention(apply_rope_pairs(q, cos, sin), apply_rope_pairs(k, cos, sin), v).reshape(B, N, D)
        x = (x.float() + _apply(self.o, a).float() * m[2][:, None]).to(x.dtype)
        h = torch.nn.functional.layer_norm(x.float(), (D,), self.norm3_w.float(), self.norm3_b.float(), 1e-6).to(x.dtype)
        q = _rms(_apply(self.cq, h), self.norm_cq).view(B, N, H, -1)
        k = _rms(_apply(self.ck, ctx), self.norm_ck).view(B, ctx.shape[1], H, -1)
        v = _apply(self.cv, ctx).view(B, ctx.shape[1], H, -1)
        x = x + _apply(self.co, _sdpa(q, k, v).reshape(B, N, D))
        h = (_ln(x) * (1 + m[4][:, None]) + m[3][:, None]).to(x.dtype)
        f = _apply(self.ffn_out, torch.nn.functional.gelu(_apply(self.ffn_in, h), approximate="tanh"))
        return (x.float() + f.float() * m[5][:, None]).to(x.dtype)


class WanTransformer3DModel(nn.Module):
    """`config`: in_channels, out_channels, patch_size (pt, ph, pw), num_attention_heads,
    attention_head_dim, ffn_dim, num_layers, text_dim, freq_dim."""

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        c = config
        self.config = c
        self.dim = c.num_attention_heads * c.attention_head_dim
        self.patch = tuple(c.patch_size)
        pin = c.in_channels * math.prod(self.patch)
        self.patch_embedding = _lin(self.dim, pin, dtype)
        self.text_in, self.text_out = _lin(self.dim, c.text_dim, dtype), _lin(self.dim, self.dim, dtype)
        self.time_in, self.time_out = _lin(self.dim, c.freq_dim, dtype), _lin(self.dim, self.dim, dtype)
        self.time_proj = _lin(6 * self.dim, self.dim, dtype)
        self.blocks = nn.ModuleList([WanBlock(self.dim, c.num_attention_heads, c.ffn_dim, dtype)
                                     for _ in range(c.num_layers)])
        self.head = _lin(c.out_channels * math.prod(self.patch), self.dim, dtype)
        self.head_modulation = nn.Parameter(torch.zeros(1, 2, self.dim, dtype=dtype), requires_grad=False)

    @torch.inference_mode()
    def forward(self, latents: torch.Tensor, timestep: torch.Tensor, text: torch.Tensor) -> torch.Tensor:
        """`latents [B, C, T, H, W]`, `timestep [B]`, `text [B, L, text_dim]` -> velocity like latents."""
        B, C, T, H, W = latents.shape
        pt, ph, pw = self.patch
        gt, gh, gw = T // pt, H // ph, W // pw
        x = latents.view(B, C, gt, pt, gh, ph, gw, pw).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, gt * gh * gw, -1)
        x = _apply(self.patch_embedding, x.to(self.patch_embedding.weight.dtype))
        cos, sin = rope_3d((gt, gh, gw), self.config.attention_head_dim, x.device)
        te = timestep_embedding(timestep, self.config.freq_dim).to(x.dtype)
        e = _apply(self.time_out, torch.nn.functional.silu(_apply(self.time_in, te)))
        e6 = _apply(self.time_proj, torch.nn.functional.silu(e)).view(B, 6, self.dim)
        ctx = _apply(self.text_out, torch.nn.functional.gelu(_apply(self.text_in, text.to(x.dtype)), approximate="tanh"))
        for blk in self.blocks:
            x = blk(x, ctx, e6, cos, sin)
        m = (self.head_modulation.float() + e.float()[:, None]).unbind(1)
        x = (_ln(x) * (1 + m[1][:, None]) + m[0][:, None]).to(x.dtype)
        x = _apply(self.head, x)
        co = self.config.out_channels
        return x.view(B, gt, gh, gw, co, pt, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7).reshape(B, co, T, H, W)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            if name in params:
                params[name].data.copy_(w.to(params[name].dtype).reshape(params[name].shape))
                loaded.add(name)
        return loaded


EntryClass = [WanTransformer3DModel]
