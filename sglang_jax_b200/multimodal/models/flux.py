"""Flux image DiT (reference `python/sgl_jax/srt/multimodal/models/dits/flux.py`): `num_layers`
double-stream blocks in which image and text tokens keep separate weights but attend jointly,
then `num_single_layers` single-stream blocks over the concatenated sequence (attention and MLP
in parallel, one fused output projection).  Conditioning is adaLN from timestep (+ guidance for
the distilled checkpoints) and the pooled CLIP vector; positions are rotary over
`axes_dims_rope` bands indexed by (0, row, col), text tokens at the origin.

Parameter names follow the published checkpoint (`x_embedder`, `context_embedder`,
`time_text_embed.*`, `transformer_blocks.N.*`, `single_transformer_blocks.N.*`, `norm_out.linear`,
`proj_out`).  Latents are packed 2x2 into `in_channels = 4 * vae_channels` tokens."""

from __future__ import annotations

import math
from typing import Iterable

import torch
import torch.nn.functional as F
from torch import nn

from .dit import _apply, _lin, _ln, _rms, apply_rope_pairs


def sinusoid(t: torch.Tensor, dim: int = 256) -> torch.Tensor:
    """(cos, sin) timestep features, frequencies `10000^(-i/half)`."""
    half = dim // 2
    f = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    a = t.float()[:, None] * f[None]
    return torch.cat([a.cos(), a.sin()], dim=-1)


def rope_nd(ids: torch.Tensor, axes_dims: tuple[int, ...], theta: float = 10000.0):
    """`ids [S, n_axes]` -> cos/sin `[S, sum(axes_dims)/2]`, one band of frequencies per axis."""
    out = []
    for i, d in enumerate(axes_dims):
        inv = 1.0 / theta ** (torch.arange(0, d, 2, dtype=torch.float32, device=ids.device) / d)
        out.append(ids[:, i].float()[:, None] * inv[None])
    ang = torch.cat(out, dim=-1)
    return ang.cos(), ang.sin()


class _MLPEmbed(nn.Module):
    def __init__(self, i, o, dtype):
        super().__init__()
        self.linear_1, self.linear_2 = _lin(o, i, dtype), _lin(o, o, dtype)

    def forward(self, x):
        return _apply(self.linear_2, F.silu(_apply(self.linear_1, x)))


class _TimeTextEmbed(nn.Module):
    def __init__(self, dim, pooled_dim, guidance: bool, dtype):
        super().__init__()
        self.timestep_embedder = _MLPEmbed(256, dim, dtype)
        self.guidance_embedder = _MLPEmbed(256, dim, dtype) if guidance else None
        self.text_embedder = _MLPEmbed(pooled_dim, dim, dtype)

    def forward(self, t, guidance, pooled):
        dt = self.timestep_embedder.linear_1.weight.dtype
        e = self.timestep_embedder(sinusoid(t).to(dt))
        if self.guidance_embedder is not None:
            e = e + self.guidance_embedder(sinusoid(guidance).to(dt))
        return e + self.text_embedder(pooled.to(dt))


class _Attn(nn.Module):
    """Joint attention.  With `context=True` the text stream has its own q/k/v/out projections."""

    def __init__(self, dim, heads, dtype, context: bool, out_proj: bool):
        super().__init__()
        self.heads = heads
        hd = dim // heads
        self.to_q, self.to_k, self.to_v = (_lin(dim, dim, dtype) for _ in range(3))
        self.norm_q, self.norm_k = nn.Module(), nn.Module()
        for m in (self.norm_q, self.norm_k):
            m.weight = nn.Parameter(torch.ones(hd, dtype=dtype), requires_grad=False)
        self.to_out = nn.ModuleList([_lin(dim, dim, dtype)]) if out_proj else None
        self.context = context
        if context:
            self.add_q_proj, self.add_k_proj, self.add_v_proj = (_lin(dim, dim, dtype) for _ in range(3))
            self.norm_added_q, self.norm_added_k = nn.Module(), nn.Module()
            for m in (self.norm_added_q, self.norm_added_k):
                m.weight = nn.Parameter(torch.ones(hd, dtype=dtype), requires_grad=False)
            self.to_add_out = _lin(dim, dim, dtype)

    def _qkv(self, x, pq, pk, pv, nq, nk):
        B, S, D = x.shape
        sh = (B, S, self.heads, D // self.heads)
        return _rms(_apply(pq, x).view(sh), nq.weight), _rms(_apply(pk, x).view(sh), nk.weight), _apply(pv, x).view(sh)

    def forward(self, x, ctx, cos, sin):
        q, k, v = self._qkv(x, self.to_q, self.to_k, self.to_v, self.norm_q, self.norm_k)
        L = 0
        if ctx is not None:
            cq, ck, cv = self._qkv(ctx, self.add_q_proj, self.add_k_proj, self.add_v_proj, self.norm_added_q,
                                   self.norm_added_k)
            L = ctx.shape[1]
            q, k, v = torch.cat([cq, q], 1), torch.cat([ck, k], 1), torch.cat([cv, v], 1)
        q, k = apply_rope_pairs(q, cos, sin), apply_rope_pairs(k, cos, sin)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
        o = o.reshape(o.shape[0], o.shape[1], -1)
        if ctx is None:
            return o if self.to_out is None else _apply(self.to_out[0], o)
        return _apply(self.to_out[0], o[:, L:]), _apply(self.to_add_out, o[:, :L])


class _FF(nn.Module):
    def __init__(self, dim, dtype):
        super().__init__()
        first = nn.Module()
        first.proj = _lin(4 * dim, dim, dtype)
        self.net = nn.ModuleList([first, nn.Identity(), _lin(dim, 4 * dim, dtype)])

    def forward(self, x):
        return _apply(self.net[2], F.gelu(_apply(self.net[0].proj, x), approximate="tanh"))


def _ada(linear, temb, n):
    return _apply(linear, F.silu(temb)).float().chunk(n, dim=-1)


def _mod(x, shift, scale):
    return (_ln(x).float() * (1 + scale[:, None]) + shift[:, None]).to(x.dtype)


class FluxDoubleBlock(nn.Module):
    def __init__(self, dim, heads, dtype):
        super().__init__()
        self.norm1, self.norm1_context = nn.Module(), nn.Module()
        self.norm1.linear, self.norm1_context.linear = _lin(6 * dim, dim, dtype), _lin(6 * dim, dim, dtype)
        self.attn = _Attn(dim, heads, dtype, context=True, out_proj=True)
        self.ff, self.ff_context = _FF(dim, dtype), _FF(dim, dtype)

    def forward(self, x, ctx, temb, cos, sin):
        sa, ca, ga, sm, cm, gm = _ada(self.norm1.linear, temb, 6)
        csa, cca, cga, csm, ccm, cgm = _ada(self.norm1_context.linear, temb, 6)
        a, c = self.attn(_mod(x, sa, ca), _mod(ctx, csa, cca), cos, sin)
        x = (x.float() + ga[:, None] * a.float()).to(x.dtype)
        x = (x.float() + gm[:, None] * self.ff(_mod(x, sm, cm)).float()).to(x.dtype)
        ctx = (ctx.float() + cga[:, None] * c.float()).to(ctx.dtype)
        ctx = (ctx.float() + cgm[:, None] * self.ff_context(_mod(ctx, csm, ccm)).float()).to(ctx.dtype)
        return x, ctx


class FluxSingleBlock(nn.Module):
    def __init__(self, dim, heads, dtype):
        super().__init__()
        self.norm = nn.Module()
        self.norm.linear = _lin(3 * dim, dim, dtype)
        self.proj_mlp = _lin(4 * dim, dim, dtype)
        self.attn = _Attn(dim, heads, dtype, context=False, out_proj=False)
        self.proj_out = _lin(dim, 5 * dim, dtype)

    def forward(self, h, temb, cos, sin):
        shift, scale, gate = _ada(self.norm.linear, temb, 3)
        n = _mod(h, shift, scale)
        y = torch.cat([self.attn(n, None, cos, sin), F.gelu(_apply(self.proj_mlp, n), approximate="tanh")], dim=-1)
        return (h.float() + gate[:, None] * _apply(self.proj_out, y).float()).to(h.dtype)


class FluxTransformer2DModel(nn.Module):
    """`config`: in_channels (64), num_layers (19), num_single_layers (38), attention_head_dim (128),
    num_attention_heads (24), joint_attention_dim (4096), pooled_projection_dim (768),
    guidance_embeds, axes_dims_rope ((16, 56, 56))."""

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        c = config
        self.config = c
        H, hd = c.num_attention_heads, c.attention_head_dim
        self.dim = dim = H * hd
        self.axes = tuple(getattr(c, "axes_dims_rope", None) or (hd // 8, hd * 7 // 16, hd * 7 // 16))
        assert sum(self.axes) == hd, "rotary bands must cover the head"
        self.patch = (1, 2, 2)
        self.vae_channels = c.in_channels // 4
        self.x_embedder = _lin(dim, c.in_channels, dtype)
        self.context_embedder = _lin(dim, c.joint_attention_dim, dtype)
        self.time_text_embed = _TimeTextEmbed(dim, getattr(c, "pooled_projection_dim", 768),
                                              bool(getattr(c, "guidance_embeds", False)), dtype)
        self.transformer_blocks = nn.ModuleList([FluxDoubleBlock(dim, H, dtype) for _ in range(c.num_layers)])
        self.single_transformer_blocks = nn.ModuleList([FluxSingleBlock(dim, H, dtype)
                                                        for _ in range(getattr(c, "num_single_layers", 0))])
        self.norm_out = nn.Module()
        self.norm_out.linear = _lin(2 * dim, dim, dtype)
        self.proj_out = _lin(getattr(c, "out_channels", None) or c.in_channels, dim, dtype)

    @torch.inference_mode()
    def forward(self, latents, timestep, text, pooled=None, guidance=None):
        """`latents [B, C, 1, H, W]` (C = in_channels / 4), `timestep [B]` on the 0..1000 scale,
        `text [B, L, joint_attention_dim]`, `pooled [B, pooled_projection_dim]` -> velocity like latents."""
        B, C, T, Hh, W = latents.shape
        gh, gw = Hh // 2, W // 2
        x = latents.view(B, C, gh, 2, gw, 2).permute(0, 2, 4, 1, 3, 5).reshape(B, gh * gw, C * 4)
        dt = self.x_embedder.weight.dtype
        x = _apply(self.x_embedder, x.to(dt))
        ctx = _apply(self.context_embedder, text.to(dt))
        L = ctx.shape[1]
        if pooled is None:
            pooled = torch.zeros(B, self.time_text_embed.text_embedder.linear_1.weight.shape[1], device=x.device)
        if guidance is None:
            guidance = torch.full((B,), 3.5, device=x.device)
        temb = self.time_text_embed(timestep, guidance.float() * 1000.0, pooled)
        ids = torch.zeros(L + gh * gw, 3, device=x.device)
        ids[L:, 1] = torch.arange(gh, device=x.device).repeat_interleave(gw)
        ids[L:, 2] = torch.arange(gw, device=x.device).repeat(gh)
        cos, sin = rope_nd(ids, self.axes)
        for blk in self.transformer_blocks:
            x, ctx = blk(x, ctx, temb, cos, sin)
        h = torch.cat([ctx, x], dim=1)
        for blk in self.single_transformer_blocks:
            h = blk(h, temb, cos, sin)
        x = h[:, L:]
        scale, shift = _ada(self.norm_out.linear, temb, 2)
        x = _apply(self.proj_out, _mod(x, shift, scale))
        return x.view(B, gh, gw, C, 2, 2).permute(0, 3, 1, 4, 2, 5).reshape(B, C, 1, Hh, W)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            if name in params:
                params[name].data.copy_(w.to(params[name].dtype).reshape(params[name].shape))
                loaded.add(name)
        return loaded


EntryClass = [FluxTransformer2DModel]
