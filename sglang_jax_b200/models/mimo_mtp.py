"""MiMo multi-token-prediction draft layers (NEXTN speculative decoding).

Each MTP layer is `input_proj(cat(token_layernorm(embed(token)), hidden_layernorm(hidden)))`
followed by one Qwen2 decoder layer and a final norm; the embedding table and LM head are
the target model's.  Layer `j` owns KV layer `j`.  Which layer runs is chosen by
`forward_batch.spec_info.mtp_layer` (default 0); `mtp_all_layers=True` runs every layer on
the same inputs (used when caches are populated) and returns layer 0's logits.

Reference: `python/sgl_jax/srt/models/mimo_mtp.py`,
`python/sgl_jax/srt/speculative/multi_layer_draft_worker.py`.
"""

from __future__ import annotations

from typing import Iterable

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding
from ..layers.layernorm import RMSNorm
from ..layers.linear import ReplicatedLinear
from ..layers.logits_processor import LogitsProcessor
from .llama import DenseAttention, DenseMLP


class MiMoMTPLayer(nn.Module):
    def __init__(self, config, layer_id: int, dtype):
        super().__init__()
        H = config.hidden_size
        eps = getattr(config, "rms_norm_eps", 1e-6)
        self.token_layernorm = RMSNorm(H, eps, dtype)
        self.hidden_layernorm = RMSNorm(H, eps, dtype)
        self.input_proj = ReplicatedLinear(2 * H, H, False, dtype)
        self.input_layernorm = RMSNorm(H, eps, dtype)
        self.self_attn = DenseAttention(config, layer_id, dtype, qkv_bias=True, o_bias=False)
        self.post_attention_layernorm = RMSNorm(H, eps, dtype)
        self.mlp = DenseMLP(H, config.intermediate_size, dtype)
        self.final_layernorm = RMSNorm(H, eps, dtype)

    def forward(self, emb, hidden, forward_batch):
        x = self.input_proj(torch.cat([self.token_layernorm(emb), self.hidden_layernorm(hidden)], dim=-1))
        residual = x
        a = self.self_attn.o_proj(self.self_attn(self.input_layernorm(x), forward_batch))
        residual = residual + a
        out = residual + self.mlp(self.post_attention_layernorm(residual))
        return self.final_layernorm(out)


class _MTPModel(nn.Module):
    def __init__(self, config, dtype, n_layers):
        super().__init__()
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        self.mtp_layers = nn.ModuleList([MiMoMTPLayer(config, j, dtype) for j in range(n_layers)])


class MiMoMTP(nn.Module):
    is_eagle_draft = True
    share_lm_head = True
    stacked_params_mapping = [
        (".qkv_proj", ".q_proj", "q"), (".qkv_proj", ".k_proj", "k"), (".qkv_proj", ".v_proj", "v"),
        (".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1),
    ]

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        self.config = config
        n = int(getattr(config, "num_nextn_predict_layers", 1) or 1)
        self.num_mtp_layers = n
        self.num_kv_layers = n
        self.model = _MTPModel(config, dtype, n)
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.logits_processor = LogitsProcessor(config.vocab_size)
        self._loaded: set = set()

    def get_embed_and_head(self):
        return self.model.embed_tokens.weight, self.lm_head.weight

    def set_embed_and_head(self, embed, head):
        self.model.embed_tokens.weight = nn.Parameter(embed, requires_grad=False)
        if head is not None:
            self.lm_head.weight = nn.Parameter(head, requires_grad=False)

    def forward(self, input_ids, forward_batch, input_embeds=None):
        si = forward_batch.spec_info
        emb = self.model.embed_tokens(input_ids)
        hidden = si.hidden_states.to(emb.dtype)
        if getattr(si, "mtp_all_layers", False):
            outs = [layer(emb, hidden, forward_batch) for layer in self.model.mtp_layers]
            h = outs[0]
        else:
            j = min(int(getattr(si, "mtp_layer", 0) or 0), self.num_mtp_layers - 1)
            h = self.model.mtp_layers[j](emb, hidden, forward_batch)
        out = self.logits_processor(h, self.lm_head, forward_batch)
        if forward_batch.capture_hidden_mode:
            out.hidden_states = h if forward_batch.capture_hidden_mode == 2 or forward_batch.last_token_indices is None \
                else h[forward_batch.last_token_indices]
        return out

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        modules = dict(self.named_modules())
        loaded = set()
        for name, w in weights:
            if "mtp_layers" not in name:
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
        return loaded | {"model.embed_tokens.weight", "lm_head.weight"}


class MiMoMTPForCausalLM(MiMoMTP):
    """Name under which the reference registers the MiMo MTP draft model (`models/mimo_mtp.py` `EntryClass`)."""


EntryClass = [MiMoMTP, MiMoMTPForCausalLM]
