"""DFlash block-diffusion draft model.

The draft owns neither an embedding table nor an LM head (both are the target's).  Its KV
cache over the *context* is not produced by running the draft: it is projected from target
hidden features (`materialize_kv`: the features of a few target layers are concatenated,
mapped by `fc`, normalised, and pushed through every draft layer's k/v projections).  One
draft forward then denoises a whole block `[anchor, MASK, ..., MASK]` at once with
bidirectional attention inside the block.

Reference: `python/sgl_jax/srt/models/dflash.py`.
"""

from __future__ import annotations

from typing import Iterable

import torch
from torch import nn

from .. import ops
from ..layers.layernorm import RMSNorm
from ..layers.linear import ReplicatedLinear
from ..ops import reference
from .llama import DenseAttention, DenseMLP


class DFlashDecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype):
        super().__init__()
        eps = getattr(config, "rms_norm_eps", 1e-6)
        self.input_layernorm = RMSNorm(config.hidden_size, eps, dtype)
        self.self_attn = DenseAttention(config, layer_id, dtype, qkv_bias=getattr(config, "attention_bias", False),
                                        o_bias=getattr(config, "attention_bias", False), qk_norm=True)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps, dtype)
        self.mlp = DenseMLP(config.hidden_size, config.intermediate_size, dtype)

    def forward(self, x, forward_batch):
        a = self.self_attn.o_proj(self.self_attn(self.input_layernorm(x), forward_batch))
        x = x + a
        return x + self.mlp(self.post_attention_layernorm(x))


class _Backbone(nn.Module):
    def __init__(self, config, dtype):
        super().__init__()
        self.layers = nn.ModuleList([DFlashDecoderLayer(config, i, dtype) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, getattr(config, "rms_norm_eps", 1e-6), dtype)


class DFlashDraftModel(nn.Module):
    stacked_params_mapping = [
        (".qkv_proj", ".q_proj", "q"), (".qkv_proj", ".k_proj", "k"), (".qkv_proj", ".v_proj", "v"),
        (".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1),
    ]
    is_dflash_draft = True

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        self.config = config
        H = config.hidden_size
        dcfg = getattr(config, "dflash_config", None) or {}
        ids = getattr(config, "target_layer_ids", None) or dcfg.get("target_layer_ids")
        self.target_layer_ids = list(ids) if ids is not None else None
        n_feat = len(ids) if ids is not None else int(config.num_hidden_layers)
        self.num_context_features = n_feat
        self.target_hidden_size = int(getattr(config, "target_hidden_size", None) or H)
        self.block_size = int(getattr(config, "block_size", None) or dcfg.get("block_size", 4))
        self.mask_token_id = int(getattr(config, "mask_token_id", None) or dcfg.get("mask_token_id", 0))
        self.model = _Backbone(config, dtype)
        self.fc = ReplicatedLinear(n_feat * self.target_hidden_size, H, False, dtype)
        self.hidden_norm = RMSNorm(H, getattr(config, "rms_norm_eps", 1e-6), dtype)
        self.embed_weight: torch.Tensor | None = None
        self.head_weight: torch.Tensor | None = None

    def set_embed_and_head(self, embed, head):
        self.embed_weight, self.head_weight = embed, head

    def project_target_hidden(self, target_hidden: torch.Tensor) -> torch.Tensor:
        want = self.num_context_features * self.target_hidden_size
        if target_hidden.shape[-1] != want:
            raise ValueError(f"DFLASH target feature width {target_hidden.shape[-1]} != {want}")
        return self.hidden_norm(self.fc(target_hidden.to(self.fc.weight.dtype)))

    @torch.inference_mode()
    def materialize_kv(self, target_hidden, positions, out_cache_loc, forward_batch):
        """Write the draft K/V of context tokens straight from target features."""
        ctx = self.project_target_hidden(target_hidden)
        pool = forward_batch.token_to_kv_pool
        native_backend = getattr(forward_batch.attn_backend, "name", "fa") == "native"
        rope = reference.rope_qknorm_kvwrite if native_backend else ops.rope_qknorm_kvwrite
        for layer in self.model.layers:
            a = layer.self_attn
            qkv = a.qkv_proj(ctx)
            rope(qkv, positions, a.rotary_emb.cos_sin_cache, a.q_norm.weight, a.k_norm.weight,
                 a.q_norm.variance_epsilon, a.attn.num_heads, a.attn.num_kv_heads, a.head_dim,
                 pool.get_kv_buffer(a.attn.layer_id), out_cache_loc, forward_batch.page_size,
                 a.rotary_emb.is_neox_style, a.rotary_emb.rotary_dim, False)

    def forward(self, input_ids, forward_batch, input_embeds=None):
        from ..layers.logits_processor import LogitsProcessorOutput
        x = input_embeds if input_embeds is not None else ops.embedding(input_ids, self.embed_weight)
        for layer in self.model.layers:
            x = layer(x, forward_batch)
        h = self.model.norm(x)
        logits = ops.linear(h, self.head_weight)[:, : self.config.vocab_size]
        return LogitsProcessorOutput(next_token_logits=logits, hidden_states=h)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        modules = dict(self.named_modules())
        loaded = set()
        for name, w in weights:
            if name.startswith("layers.") or name.startswith("norm."):
                name = "model." + name
            target, shard = name, None
            for pfrag, cfrag, sid in self.stacked_params_mapping:
                if cfrag in name:
                    target, shard = name.replace(cfrag, pfrag), sid
                    break
            if target not in params:
                continue
            mod = modules[target.rsplit(".", 1)[0]]
            p = params[target]
            mod.weight_loader(p, w.to(p.dtype) if w.dtype != p.dtype else w, shard)
            loaded.add(target)
        return loaded


EntryClass = [DFlashDraftModel]
