"""MiMo-Audio backbone (reference
`python/sgl_jax/srt/multimodal/models/mimo_audio/mimo_audio_backbone.py`).

The language model steps over *groups* of `group_size` audio frames.  A group's input embedding
is the text-token embedding plus `speech_group_downcast(patch_encoder(sum over channels of the
codebook embeddings))` — the patch encoder is a small bidirectional transformer over the frames
of one group.  After each language-model step the text head picks a token; when it is the
`empty` marker the step is speech, and a small causal *patch decoder* generates the group's
`group_size x audio_channels` codes from `hidden_states_downcast(hidden)` — one frame per local
step, channel `c` delayed by `delay_pattern[c]` steps, with its keys and values cached across the
local steps.

The main transformer is a Qwen2 decoder served by the regular model runner; this module holds
the local transformers and heads (checkpoint names `input_local_transformer.*`,
`local_transformer.*`, `speech_embeddings.N`, `local_transformer_lm_heads.N`,
`speech_group_downcast`, `hidden_states_downcast`)."""

from __future__ import annotations

from typing import Iterable

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from ...ops import reference


def _lin(x, lin):
    return ops.linear(x.reshape(-1, x.shape[-1]), lin.weight, lin.bias).view(*x.shape[:-1], -1)


class _LocalLayer(nn.Module):
    def __init__(self, dim, heads, head_dim, ffn, eps, bias, dtype):
        super().__init__()
        self.heads, self.hd, self.eps = heads, head_dim, eps
        at = nn.Module()
        at.q_proj = nn.Linear(dim, heads * head_dim, bias=bias, dtype=dtype)
        at.k_proj = nn.Linear(dim, heads * head_dim, bias=bias, dtype=dtype)
        at.v_proj = nn.Linear(dim, heads * head_dim, bias=bias, dtype=dtype)
        at.o_proj = nn.Linear(heads * head_dim, dim, bias=False, dtype=dtype)
        self.self_attn = at
        mlp = nn.Module()
        mlp.gate_proj, mlp.up_proj = nn.Linear(dim, ffn, bias=False, dtype=dtype), nn.Linear(dim, ffn, bias=False, dtype=dtype)
        mlp.down_proj = nn.Linear(ffn, dim, bias=False, dtype=dtype)
        self.mlp = mlp
        self.input_layernorm = nn.Module()
        self.post_attention_layernorm = nn.Module()
        for m in (self.input_layernorm, self.post_attention_layernorm):
            m.weight = nn.Parameter(torch.ones(dim, dtype=dtype))

    def forward(self, x, positions, cos_sin, causal, cache):
        B, T, _ = x.shape
        h = reference.rmsnorm(x, self.input_layernorm.weight, self.eps)
        a = self.self_attn
        q, k, v = (_lin(h, p).view(B * T, self.heads, self.hd) for p in (a.q_proj, a.k_proj, a.v_proj))
        pos = positions.repeat(B)
        q = reference.apply_rope(q, pos, cos_sin, True).view(B, T, self.heads, self.hd).transpose(1, 2)
        k = reference.apply_rope(k, pos, cos_sin, True).view(B, T, self.heads, self.hd).transpose(1, 2)
        v = v.view(B, T, self.heads, self.hd).transpose(1, 2)
        if cache is not None:                       # step mode: earlier local steps stay visible
            if cache:
                k, v = torch.cat([cache[0], k], 2), torch.cat([cache[1], v], 2)
            cache[:] = [k, v]
        o = F.scaled_dot_product_attention(q, k, v, is_causal=causal and T > 1)
        x = x + _lin(o.transpose(1, 2).reshape(B, T, -1), a.o_proj)
        h = reference.rmsnorm(x, self.post_attention_layernorm.weight, self.eps)
        return x + _lin(F.silu(_lin(h, self.mlp.gate_proj)) * _lin(h, self.mlp.up_proj), self.mlp.down_proj)


class LocalTransformer(nn.Module):
    def __init__(self, dim, layers, heads, head_dim, ffn, theta, eps, bias, causal, max_pos, dtype):
        super().__init__()
        self.causal = causal
        self.layers = nn.ModuleList([_LocalLayer(dim, heads, head_dim, ffn, eps, bias, dtype) for _ in range(layers)])
        self.norm = nn.Module()
        self.norm.weight = nn.Parameter(torch.ones(dim, dtype=dtype))
        self.eps = eps
        inv = 1.0 / theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim)
        ang = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv[None]
        self.register_buffer("cos_sin", torch.cat([ang.cos(), ang.sin()], dim=-1), persistent=False)

    def forward(self, x, positions, caches=None):
        for i, layer in enumerate(self.layers):
            x = layer(x, positions, self.cos_sin, self.causal, None if caches is None else caches[i])
        return reference.rmsnorm(x, self.norm.weight, self.eps)


class MiMoAudioLocalModules(nn.Module):
    """Everything of the backbone except the main transformer."""

    def __init__(self, config, dtype=torch.bfloat16):
        super().__init__()
        c = config
        self.config = c
        self.group, self.channels = c.group_size, c.audio_channels
        self.vocab_sizes = list(c.speech_vocab_sizes)
        self.empty_ids = list(c.speech_empty_ids)
        self.delay = list(getattr(c, "delay_pattern", None) or [0] * self.channels)
        bias = bool(getattr(c, "attention_bias", True))
        local_pos = max(64, self.group + max(self.delay) + 1)
        self.local_transformer = LocalTransformer(c.local_dim, c.local_layers, c.local_attn_heads, c.local_head_dim,
                                                  c.local_ffn_dim, c.rope_theta, c.rms_norm_eps, bias, True, local_pos, dtype)
        self.input_local_transformer = LocalTransformer(c.input_local_dim, c.input_local_layers, c.local_attn_heads,
                                                        c.local_head_dim, c.local_ffn_dim, c.rope_theta, c.rms_norm_eps,
                                                        bias, not getattr(c, "input_full_attention", True), local_pos, dtype)
        self.speech_embeddings = nn.ModuleList([nn.Embedding(v, c.input_local_dim, dtype=dtype) for v in self.vocab_sizes])
        self.local_transformer_lm_heads = nn.ModuleList([nn.Linear(c.local_dim, v, bias=False, dtype=dtype)
                                                         for v in self.vocab_sizes])
        self.speech_group_downcast = nn.Linear(c.input_local_dim * self.group, c.hidden_size, bias=False, dtype=dtype)
        self.hidden_states_downcast = nn.Linear(c.hidden_size, c.local_dim, bias=False, dtype=dtype)
        for p in self.parameters():
            p.requires_grad_(False)

    @torch.inference_mode()
    def group_embeds(self, speech_ids: torch.Tensor, is_speech: torch.Tensor) -> torch.Tensor:
        """`speech_ids [G, group, channels]`, `is_speech bool [G]` -> the speech part of the groups'
        language-model input embeddings `[G, hidden]` (zero rows for text groups)."""
        G = speech_ids.shape[0]
        e = 0
        for c in range(self.channels):
            ids = speech_ids[..., c]
            emb = self.speech_embeddings[c](ids.clamp_max(self.vocab_sizes[c] - 1))
            e = e + emb * (ids != self.empty_ids[c])[..., None]
        e = e * is_speech[:, None, None]
        e = self.input_local_transformer(e, torch.arange(self.group, device=e.device))
        e = e * is_speech[:, None, None]
        return _lin(e.reshape(G, -1), self.speech_group_downcast)

    @torch.inference_mode()
    def patch_decode(self, hidden: torch.Tensor, temperature: float = 0.0, generator=None) -> torch.Tensor:
        """`hidden [B, hidden]` (language-model output of a speech step) -> codes `[B, group, channels]`."""
        B = hidden.shape[0]
        x = _lin(hidden, self.hidden_states_downcast)[:, None, :]
        tokens = torch.zeros(B, self.group, self.channels, dtype=torch.long, device=hidden.device)
        caches = [[] for _ in self.local_transformer.layers]
        for t in range(self.group + max(self.delay)):
            h = self.local_transformer(x, torch.tensor([t], device=x.device), caches)[:, -1]
            nxt = torch.zeros_like(x)
            for c in range(self.channels):
                s = self.delay[c]
                if not (s <= t < s + self.group):
                    continue
                logits = _lin(h, self.local_transformer_lm_heads[c]).float()
                logits[:, self.empty_ids[c]] = float("-inf")
                if temperature > 1e-6:
                    tok = torch.multinomial(torch.softmax(logits / temperature, -1).cpu(), 1, generator=generator)[:, 0].to(x.device)
                else:
                    tok = logits.argmax(-1)
                tokens[:, t - s, c] = tok
                nxt = nxt + self.speech_embeddings[c](tok)[:, None, :]
            x = nxt
        return tokens

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            if name in params:
                params[name].data.copy_(w.to(params[name].dtype))
                loaded.add(name)
        return loaded


EntryClass = [MiMoAudioLocalModules]
