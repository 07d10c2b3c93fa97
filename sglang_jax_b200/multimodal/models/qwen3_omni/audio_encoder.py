"""Qwen3-Omni audio encoder (reference
`python/sgl_jax/srt/multimodal/models/qwen3_omni_moe/audio_encoder.py`).

A log-mel spectrogram `[num_mel_bins, frames]` is cut into chunks of `2 * n_window` frames; each
chunk goes through three stride-2 3x3 convolutions (8x fewer frames) and a linear map to
`d_model`, gets sinusoidal positions that restart per chunk, and the valid frames of all chunks
are packed into one sequence.  Pre-LN transformer layers attend within windows of
`n_window_infer` input frames; a LayerNorm and a two-layer head produce `output_dim` features
(one per 8 input frames... 13 per 100)."""

from __future__ import annotations

import math
from typing import Iterable

import torch
import torch.nn.functional as F
from torch import nn

from .... import ops
from ..segments import PackedSegments


def feat_lengths(n: torch.Tensor) -> torch.Tensor:
    """Frames that survive the convolution stack for `n` mel frames (13 per full 100-frame block)."""
    leave = n % 100
    f = (leave - 1) // 2 + 1
    return ((f - 1) // 2 + 1 - 1) // 2 + 1 + (n // 100) * 13


def sinusoids(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2).float())
    t = torch.arange(length)[:, None] * inv[None]
    return torch.cat([t.sin(), t.cos()], dim=1)


def _lin(x, lin):
    return ops.linear(x.reshape(-1, x.shape[-1]), lin.weight, lin.bias).view(*x.shape[:-1], -1)


class AudioEncoderLayer(nn.Module):
    def __init__(self, d, heads, ffn, act, dtype):
        super().__init__()
        self.heads = heads
        self.self_attn = nn.Module()
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            setattr(self.self_attn, n, nn.Linear(d, d, dtype=dtype))
        self.self_attn_layer_norm = nn.LayerNorm(d, dtype=dtype)
        self.final_layer_norm = nn.LayerNorm(d, dtype=dtype)
        self.fc1, self.fc2 = nn.Linear(d, ffn, dtype=dtype), nn.Linear(ffn, d, dtype=dtype)
        self.act = act

    def forward(self, x, mask):
        T, D = x.shape
        h = self.self_attn_layer_norm(x)
        a = self.self_attn
        q, k, v = (_lin(h, p).view(T, self.heads, -1) for p in (a.q_proj, a.k_proj, a.v_proj))
        x = x + _lin(mask.attend(q, k, v), a.out_proj)
        return x + _lin(self.act(_lin(self.final_layer_norm(x), self.fc1)), self.fc2)


class Qwen3OmniMoeAudioEncoder(nn.Module):
    """`config`: num_mel_bins, d_model, encoder_layers, encoder_attention_heads, encoder_ffn_dim,
    downsample_hidden_size, output_dim, max_source_positions, n_window, n_window_infer,
    activation_function."""

    def __init__(self, config, dtype=torch.bfloat16):
        super().__init__()
        c = config
        self.config = c
        d, dh = c.d_model, c.downsample_hidden_size
        self.n_window, self.n_window_infer = c.n_window, c.n_window_infer
        act = {"gelu": F.gelu, "relu": F.relu, "silu": F.silu}[getattr(c, "activation_function", "gelu")]
        self.act = act
        self.register_buffer("positional_embedding", sinusoids(c.max_source_positions, d), persistent=False)
        self.conv2d1 = nn.Conv2d(1, dh, 3, 2, padding=1, dtype=dtype)
        self.conv2d2 = nn.Conv2d(dh, dh, 3, 2, padding=1, dtype=dtype)
        self.conv2d3 = nn.Conv2d(dh, dh, 3, 2, padding=1, dtype=dtype)
        f = (((c.num_mel_bins + 1) // 2 + 1) // 2 + 1) // 2
        self.conv_out = nn.Linear(dh * f, d, bias=False, dtype=dtype)
        self.layers = nn.ModuleList([AudioEncoderLayer(d, c.encoder_attention_heads, c.encoder_ffn_dim, act, dtype)
                                     for _ in range(c.encoder_layers)])
        self.ln_post = nn.LayerNorm(d, dtype=dtype)
        self.proj1, self.proj2 = nn.Linear(d, d, dtype=dtype), nn.Linear(d, c.output_dim, dtype=dtype)
        for p in self.parameters():
            p.requires_grad_(False)

    @torch.inference_mode()
    def forward(self, input_features: torch.Tensor, feature_lens: torch.Tensor) -> torch.Tensor:
        """`input_features [num_mel_bins, sum(feature_lens)]` (clips concatenated along time) ->
        `[sum(feat_lengths(feature_lens)), output_dim]`."""
        W = self.n_window * 2
        dt = self.conv2d1.weight.dtype
        feature_lens = feature_lens.long().cpu()
        chunk_lens = []
        for n in feature_lens.tolist():
            full, rem = divmod(n, W)
            chunk_lens += [W] * full + ([rem] if rem else [])
        chunks = input_features.T.split(chunk_lens, dim=0)
        padded = nn.utils.rnn.pad_sequence(list(chunks), batch_first=True).transpose(1, 2).unsqueeze(1).to(dt)
        x = F.gelu(self.conv2d3(F.gelu(self.conv2d2(F.gelu(self.conv2d1(padded))))))
        b, ch, f, t = x.shape
        x = _lin(x.permute(0, 3, 1, 2).reshape(b, t, ch * f), self.conv_out)
        x = x + self.positional_embedding[:t].to(x.dtype)
        after = feat_lengths(torch.tensor(chunk_lens))
        keep = torch.arange(t)[None, :] < after[:, None]
        h = x[keep.to(x.device)]
        # attention windows: `n_window_infer` input frames worth of encoder frames, per clip
        window = t * (self.n_window_infer // W)
        seg = []
        for n in feat_lengths(feature_lens).tolist():
            seg += [window] * (n // window) + ([n % window] if n % window else [])
        mask = PackedSegments(seg, h.device)
        for layer in self.layers:
            h = layer(h, mask)
        return _lin(self.act(_lin(self.ln_post(h), self.proj1)), self.proj2)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            n = name.split("audio_tower.", 1)[-1]
            if n in params:
                params[n].data.copy_(w.to(params[n].dtype))
                loaded.add(n)
        return loaded


EntryClass = [Qwen3OmniMoeAudioEncoder]
