"""EAGLE / EAGLE-3 draft heads for Llama-style targets.

A draft head is a one-layer decoder that predicts token i+2 from the pair
(token i+1, target hidden state i).  It shares the request rows and KV slot indices
with the target model and owns a single KV layer.

* `LlamaForCausalLMEagle` (EAGLE-1/2): `fc(cat(embed(token), hidden))` -> decoder layer
  without input norm -> shared LM head.
* `LlamaForCausalLMEagle3`: the hidden input is the concatenation of three target layers
  (`fc` maps 3H -> H on the first step; later steps feed the head's own output), the
  decoder layer attends over `cat(norm(embed), norm(hidden))` (2H-wide qkv input), and
  the head has its own reduced vocabulary with a `d2t` offset table.

Reference: `python/sgl_jax/srt/models/llama_eagle3.py`,
`python/sgl_jax/srt/speculative/eagle_draft_worker.py`.
"""

from __future__ import annotations

from typing import Iterable

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding
from ..layers.layernorm import RMSNorm
from ..layers.linear import QKVParallelLinear, ReplicatedLinear
from ..layers.logits_processor import LogitsProcessor
from .llama import DenseAttention, DenseMLP


def _draft_hidden(forward_batch, like: torch.Tensor) -> torch.Tensor:
    si = forward_batch.spec_info
    hs = getattr(si, "hidden_states", None) if si is not None else None
    if hs is None:
        raise RuntimeError("an EAGLE draft head needs spec_info.hidden_states")
    return hs.to(like.dtype)


class _EagleLayer(nn.Module):
    def __init__(self, config, dtype, qkv_in: int | None = None, input_norm: bool = False):
        super().__init__()
        eps = getattr(config, "rms_norm_eps", 1e-6)
        self.self_attn = DenseAttention(config, 0, dtype, qkv_bias=getattr(config, "attention_bias", False),
                                        o_bias=getattr(config, "attention_bias", False))
        if qkv_in is not None:
            a = self.self_attn
            a.qkv_proj = QKVParallelLinear(qkv_in, a.head_dim, a.total_heads, a.total_kv_heads,
                                           getattr(config, "attention_bias", False), dtype)
        self.mlp = DenseMLP(config.hidden_size, config.intermediate_size, dtype, getattr(config, "mlp_bias", False))
        self.input_layernorm = RMSNorm(config.hidden_size, eps, dtype) if input_norm else None
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps, dtype)


class _EagleBase(nn.Module):
    stacked_params_mapping = [
        (".qkv_proj", ".q_proj", "q"), (".qkv_proj", ".k_proj", "k"), (".qkv_proj", ".v_proj", "v"),
        (".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1),
    ]
    num_kv_layers = 1
    is_eagle_draft = True

    def get_embed_and_head(self):
        return self.model.embed_tokens.weight, self.lm_head.weight

    def set_embed_and_head(self, embed: torch.Tensor, head: torch.Tensor | None):
        """Share the target's tables (EAGLE checkpoints usually ship without them)."""
        if "model.embed_tokens.weight" not in self._loaded:
            self.model.embed_tokens.weight = nn.Parameter(embed, requires_grad=False)
        if head is not None and self.share_lm_head and "lm_head.weight" not in self._loaded:
            self.lm_head.weight = nn.Parameter(head, requires_grad=False)

    def _rename(self, name: str) -> str | None:
        return name

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        buffers = dict(self.named_buffers())
        modules = dict(self.named_modules())
        loaded = set()
        for name, w in weights:
            name = self._rename(name)
            if name is None or "rotary_emb.inv_freq" in name:
                continue
            if name in buffers:
                buffers[name].copy_(w.to(buffers[name].dtype))
                loaded.add(name)
                continue
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
        self._loaded = loaded
        # tables that may legitimately be absent: they come from the target model
        optional = {"model.embed_tokens.weight"} | ({"lm_head.weight"} if self.share_lm_head else set())
        return loaded | (optional - loaded)


class _EagleModel(nn.Module):
    def __init__(self, config, dtype, eagle3: bool):
        super().__init__()
        H = config.hidden_size
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, H, dtype)
        eps = getattr(config, "rms_norm_eps", 1e-6)
        self.eagle3 = eagle3
        if eagle3:
            tgt_h = getattr(config, "target_hidden_size", None) or H
            self.fc = ReplicatedLinear(3 * tgt_h, H, getattr(config, "bias", False), dtype)
            self.midlayer = _EagleLayer(config, dtype, qkv_in=2 * H, input_norm=True)
            self.midlayer.hidden_norm = RMSNorm(H, eps, dtype)
            self.norm = RMSNorm(H, eps, dtype)
        else:
            self.fc = ReplicatedLinear(2 * H, H, getattr(config, "bias", True), dtype)
            self.layers = nn.ModuleList([_EagleLayer(config, dtype)])

    def forward(self, input_ids, forward_batch):
        emb = self.embed_tokens(input_ids)
        hs = _draft_hidden(forward_batch, emb)
        if self.eagle3:
            if hs.shape[-1] != emb.shape[-1]:
                hs = self.fc(hs)
            lyr = self.midlayer
            residual = hs
            x = torch.cat([lyr.input_layernorm(emb), lyr.hidden_norm(hs)], dim=-1)
        else:
            lyr = self.layers[0]
            x = self.fc(torch.cat([emb, hs], dim=-1))
            residual = x
        attn = lyr.self_attn.o_proj(lyr.self_attn(x, forward_batch))
        residual = residual + attn
        h = lyr.post_attention_layernorm(residual)
        out = residual + lyr.mlp(h)
        # (hidden fed to the LM head, hidden handed to the next draft step)
        return (self.norm(out), out) if self.eagle3 else (out, out)


class LlamaForCausalLMEagle(_EagleBase):
    share_lm_head = True

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        self.config = config
        self.model = _EagleModel(config, dtype, eagle3=False)
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.logits_processor = LogitsProcessor(config.vocab_size)
        self._loaded: set = set()

    def _rename(self, name):
        if name.startswith("lm_head"):
            return name
        return name if name.startswith("model.") else "model." + name

    def forward(self, input_ids, forward_batch, input_embeds=None):
        head_in, nxt = self.model(input_ids, forward_batch)
        out = self.logits_processor(head_in, self.lm_head, forward_batch)
        if forward_batch.capture_hidden_mode:
            out.hidden_states = nxt if forward_batch.capture_hidden_mode == 2 or forward_batch.last_token_indices is None \
                else nxt[forward_batch.last_token_indices]
        return out


class LlamaForCausalLMEagle3(_EagleBase):
    share_lm_head = False

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        self.config = config
        self.model = _EagleModel(config, dtype, eagle3=True)
        draft_vocab = getattr(config, "draft_vocab_size", None) or config.vocab_size
        self.draft_vocab_size = draft_vocab
        self.lm_head = ParallelLMHead(draft_vocab, config.hidden_size, dtype)
        self.logits_processor = LogitsProcessor(draft_vocab)
        # draft id -> target id offset (hot-token vocabulary)
        self.register_buffer("d2t", torch.zeros(draft_vocab, dtype=torch.int64), persistent=False)
        self.has_d2t = draft_vocab != config.vocab_size
        self._loaded = set()

    def _rename(self, name):
        if name.startswith("t2d"):
            return None
        if name.startswith(("lm_head", "d2t")):
            return name
        if name.startswith("midlayer.") or name.startswith("fc.") or name.startswith("norm.") \
                or name.startswith("embed_tokens."):
            return "model." + name
        return name

    def map_draft_ids(self, ids: torch.Tensor) -> torch.Tensor:
        return ids + self.d2t[ids] if self.has_d2t else ids

    def forward(self, input_ids, forward_batch, input_embeds=None):
        head_in, nxt = self.model(input_ids, forward_batch)
        out = self.logits_processor(head_in, self.lm_head, forward_batch)
        if forward_batch.capture_hidden_mode:
            out.hidden_states = nxt if forward_batch.capture_hidden_mode == 2 or forward_batch.last_token_indices is None \
                else nxt[forward_batch.last_token_indices]
        return out


EntryClass = [LlamaForCausalLMEagle, LlamaForCausalLMEagle3]
