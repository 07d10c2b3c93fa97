"""CLIP text and vision encoders (the second prompt encoder of the Flux pipeline; reference
`python/sgl_jax/srt/multimodal/models/encoders/clip.py`).  Pre-LN transformer with biased
projections and a quick-GELU (or GELU) MLP.  The text tower is causal and pools the hidden state
at the end-of-text token; the vision tower prepends a class token to the patch embeddings and
pools the class position."""

from __future__ import annotations

from typing import Iterable

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops


def _act(name: str):
    if name == "quick_gelu":
        return lambda x: x * torch.sigmoid(1.702 * x)
    if name in ("gelu", "gelu_new", "gelu_pytorch_tanh"):
        return (lambda x: F.gelu(x)) if name == "gelu" else (lambda x: F.gelu(x, approximate="tanh"))
    raise ValueError(f"unsupported CLIP activation {name}")


class _Linear(nn.Module):
    def __init__(self, i, o, dtype):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(o, i, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype), requires_grad=False)

    def forward(self, x):
        return ops.linear(x.reshape(-1, x.shape[-1]), self.weight, self.bias).view(*x.shape[:-1], -1)


class _LayerNorm(nn.Module):
    def __init__(self, d, eps, dtype):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(d, dtype=dtype), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        return F.layer_norm(x.float(), x.shape[-1:], self.weight.float(), self.bias.float(), self.eps).to(x.dtype)


class CLIPEncoderLayer(nn.Module):
    def __init__(self, cfg, dtype):
        super().__init__()
        D, self.H = cfg.hidden_size, cfg.num_attention_heads
        self.layer_norm1 = _LayerNorm(D, cfg.layer_norm_eps, dtype)
        self.layer_norm2 = _LayerNorm(D, cfg.layer_norm_eps, dtype)
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (_Linear(D, D, dtype) for _ in range(4))
        self.fc1, self.fc2 = _Linear(D, cfg.intermediate_size, dtype), _Linear(cfg.intermediate_size, D, dtype)
        self.act = _act(getattr(cfg, "hidden_act", "quick_gelu"))

    def forward(self, x, mask):
        B, T, D = x.shape
        h = self.layer_norm1(x)
        q, k, v = (p(h).view(B, T, self.H, D // self.H).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))
        a = F.scaled_dot_product_attention(q.float(), k.float(), v.float(), attn_mask=mask).to(x.dtype)
        x = x + self.out_proj(a.transpose(1, 2).reshape(B, T, D))
        return x + self.fc2(self.act(self.fc1(self.layer_norm2(x))))


class _Tower(nn.Module):
    prefix = ""

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            n = name.replace(self.prefix + ".encoder.layers.", "layers.").replace(self.prefix + ".", "")
            n = n.replace("self_attn.", "").replace("mlp.", "")
            n = n.replace("embeddings.", "")
            if n in params:
                params[n].data.copy_(w.reshape(params[n].shape).to(params[n].dtype))
                loaded.add(n)
        return loaded


class CLIPTextModel(_Tower):
    prefix = "text_model"

    def __init__(self, cfg, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden_size
        self.token_embedding = nn.Embedding(cfg.vocab_size, D, dtype=dtype)
        self.position_embedding = nn.Embedding(cfg.max_position_embeddings, D, dtype=dtype)
        for e in (self.token_embedding, self.position_embedding):
            e.weight.requires_grad_(False)
        self.layers = nn.ModuleList([CLIPEncoderLayer(cfg, dtype) for _ in range(cfg.num_hidden_layers)])
        self.final_layer_norm = _LayerNorm(D, cfg.layer_norm_eps, dtype)
        self.eos_token_id = getattr(cfg, "eos_token_id", 2)

    def forward(self, input_ids, attention_mask=None, return_pooled: bool = False):
        B, T = input_ids.shape
        x = self.token_embedding(input_ids) + self.position_embedding(torch.arange(T, device=input_ids.device))
        mask = torch.ones(T, T, dtype=torch.bool, device=x.device).tril().view(1, 1, T, T)
        if attention_mask is not None:
            mask = mask & attention_mask.bool().view(B, 1, 1, T)
        for layer in self.layers:
            x = layer(x, mask)
        x = self.final_layer_norm(x)
        if not return_pooled:
            return x
        if self.eos_token_id == 2:       # original checkpoints: the end-of-text token has the largest id
            pos = input_ids.argmax(-1)
        else:
            pos = (input_ids == self.eos_token_id).int().argmax(-1)
        return x, x[torch.arange(B, device=x.device), pos]

    def encode(self, input_ids, attention_mask=None):
        """Per-token embeddings; the pooled vector is available through `forward(..., return_pooled=True)`."""
        return self.forward(input_ids, attention_mask)


class CLIPVisionModel(_Tower):
    prefix = "vision_model"

    def __init__(self, cfg, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        D, P = cfg.hidden_size, cfg.patch_size
        self.class_embedding = nn.Parameter(torch.zeros(D, dtype=dtype), requires_grad=False)
        self.patch_embedding = nn.Conv2d(getattr(cfg, "num_channels", 3), D, P, P, bias=False, dtype=dtype)
        self.patch_embedding.weight.requires_grad_(False)
        n = (cfg.image_size // P) ** 2 + 1
        self.position_embedding = nn.Embedding(n, D, dtype=dtype)
        self.position_embedding.weight.requires_grad_(False)
        self.pre_layrnorm = _LayerNorm(D, cfg.layer_norm_eps, dtype)
        self.layers = nn.ModuleList([CLIPEncoderLayer(cfg, dtype) for _ in range(cfg.num_hidden_layers)])
        self.post_layernorm = _LayerNorm(D, cfg.layer_norm_eps, dtype)

    def forward(self, pixel_values, return_pooled: bool = False):
        B = pixel_values.shape[0]
        p = self.patch_embedding(pixel_values.to(self.patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)
        x = torch.cat([self.class_embedding.view(1, 1, -1).expand(B, 1, -1), p], dim=1)
        x = self.pre_layrnorm(x + self.position_embedding.weight[: x.shape[1]])
        for layer in self.layers:
            x = layer(x, None)
        if not return_pooled:
            return x
        return x, self.post_layernorm(x[:, 0])
