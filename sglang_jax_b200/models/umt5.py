"""UMT5 / T5 text encoder (the prompt encoder of the Wan video pipeline; reference
`python/sgl_jax/srt/models/umt5.py`, `multimodal/models/t5`).  Encoder-only: unscaled
dot-product attention with a learned relative-position bias (one table per layer in UMT5, shared
from layer 0 in T5), gated-GELU FFN, RMS layer norm without mean subtraction."""

from __future__ import annotations

import math
from typing import Iterable

import torch
from torch import nn

from .. import ops


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def relative_position_bucket(rel: torch.Tensor, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Bidirectional T5 bucketing of `key_pos - query_pos`."""
    nb = num_buckets // 2
    out = (rel > 0).long() * nb
    rel = rel.abs()
    max_exact = nb // 2
    small = rel < max_exact
    large = max_exact + (torch.log(rel.float().clamp_min(1) / max_exact) / math.log(max_distance / max_exact)
                         * (nb - max_exact)).long()
    large = torch.minimum(large, torch.full_like(large, nb - 1))
    return out + torch.where(small, rel, large)


class T5Block(nn.Module):
    def __init__(self, cfg, dtype, has_bias_table: bool):
        super().__init__()
        D, H, dk, F = cfg.d_model, cfg.num_heads, cfg.d_kv, cfg.d_ff
        self.H, self.dk = H, dk
        mk = lambda o, i: nn.Parameter(torch.empty(o, i, dtype=dtype), requires_grad=False)
        self.q, self.k, self.v, self.o = mk(H * dk, D), mk(H * dk, D), mk(H * dk, D), mk(D, H * dk)
        self.rel_bias = nn.Parameter(torch.empty(cfg.relative_attention_num_buckets, H, dtype=dtype),
                                     requires_grad=False) if has_bias_table else None
        self.ln0 = nn.Parameter(torch.ones(D, dtype=dtype), requires_grad=False)
        self.ln1 = nn.Parameter(torch.ones(D, dtype=dtype), requires_grad=False)
        self.gated = bool(getattr(cfg, "is_gated_act", True))
        self.wi_0 = mk(F, D)
        self.wi_1 = mk(F, D) if self.gated else None
        self.wo = mk(D, F)
        act = getattr(cfg, "dense_act_fn", "gelu_new")
        self.act = (lambda t: torch.nn.functional.gelu(t, approximate="tanh")) if "gelu" in act else torch.relu
        self.eps = cfg.layer_norm_epsilon

    def forward(self, x, bias, key_mask):
        B, T, D = x.shape
        h = _rms(x, self.ln0, self.eps).reshape(B * T, D)
        q = ops.linear(h, self.q).view(B, T, self.H, self.dk).transpose(1, 2)
        k = ops.linear(h, self.k).view(B, T, self.H, self.dk).transpose(1, 2)
        v = ops.linear(h, self.v).view(B, T, self.H, self.dk).transpose(1, 2)
        s = torch.matmul(q.float(), k.float().transpose(-1, -2)) + bias          # T5 does not scale by sqrt(d)
        if key_mask is not None:
            s = s.masked_fill(~key_mask[:, None, None, :], float("-inf"))
        a = torch.matmul(torch.softmax(s, -1), v.float()).to(x.dtype).transpose(1, 2).reshape(B * T, self.H * self.dk)
        x = x + ops.linear(a, self.o).view(B, T, D)
        h = _rms(x, self.ln1, self.eps).reshape(B * T, D)
        g = self.act(ops.linear(h, self.wi_0))
        if self.gated:
            g = g * ops.linear(h, self.wi_1)
        return x + ops.linear(g, self.wo).view(B, T, D)


class UMT5EncoderModel(nn.Module):
    per_layer_bias = True

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        self.config = config
        self.shared = nn.Parameter(torch.empty(config.vocab_size, config.d_model, dtype=dtype), requires_grad=False)
        self.blocks = nn.ModuleList([T5Block(config, dtype, self.per_layer_bias or i == 0)
                                     for i in range(config.num_layers)])
        self.final_ln = nn.Parameter(torch.ones(config.d_model, dtype=dtype), requires_grad=False)

    @torch.inference_mode()
    def encode(self, input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        """`input_ids [B, T]` -> last hidden state `[B, T, d_model]`."""
        B, T = input_ids.shape
        x = self.shared[input_ids]
        pos = torch.arange(T, device=input_ids.device)
        buckets = relative_position_bucket(pos[None, :] - pos[:, None], self.config.relative_attention_num_buckets,
                                           self.config.relative_attention_max_distance)
        mask = attention_mask.bool() if attention_mask is not None else None
        bias = None
        for blk in self.blocks:
            if blk.rel_bias is not None:
                bias = blk.rel_bias[buckets].permute(2, 0, 1).unsqueeze(0).float()     # [1, H, T, T]
            x = blk(x, bias, mask)
        return _rms(x, self.final_ln, self.config.layer_norm_epsilon)

    forward = encode

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        table = {"shared.weight": "shared", "encoder.embed_tokens.weight": "shared",
                 "encoder.final_layer_norm.weight": "final_ln"}
        sub = {"layer.0.SelfAttention.q.weight": "q", "layer.0.SelfAttention.k.weight": "k",
               "layer.0.SelfAttention.v.weight": "v", "layer.0.SelfAttention.o.weight": "o",
               "layer.0.SelfAttention.relative_attention_bias.weight": "rel_bias", "layer.0.layer_norm.weight": "ln0",
               "layer.1.DenseReluDense.wi_0.weight": "wi_0", "layer.1.DenseReluDense.wi_1.weight": "wi_1",
               "layer.1.DenseReluDense.wi.weight": "wi_0", "layer.1.DenseReluDense.wo.weight": "wo",
               "layer.1.layer_norm.weight": "ln1"}
        loaded = set()
        for name, w in weights:
            tgt = table.get(name)
            if tgt is None and name.startswith("encoder.block."):
                _, _, i, rest = name.split(".", 3)
                if rest in sub:
                    tgt = f"blocks.{i}.{sub[rest]}"
            if tgt is None or tgt not in params:
                continue
            params[tgt].data.copy_(w.to(params[tgt].dtype))
            loaded.add(tgt)
        return loaded


class T5EncoderModel(UMT5EncoderModel):
    per_layer_bias = False


EntryClass = [UMT5EncoderModel, T5EncoderModel]
