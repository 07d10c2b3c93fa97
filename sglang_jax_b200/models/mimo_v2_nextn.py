"""MiMo-V2 multi-token-prediction draft layers (NEXTN speculative decoding for MiMo-V2-Flash /
MiMo-V2-Pro).  Each layer is `eh_proj(cat(enorm(embed(token)), hnorm(hidden)))` followed by one
sliding-window attention block (the target's SWA head layout, with its sink bias) and a dense
MLP, then a final norm; the embedding table and LM head are the target's.  Layer `j` owns KV
layer `j`; `forward_batch.spec_info.mtp_layer` picks the layer, `mtp_all_layers` runs them all.

Reference: `python/sgl_jax/srt/models/mimo_v2_nextn.py`.
"""

from __future__ import annotations

from typing import Iterable

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding
from ..layers.layernorm import RMSNorm
from ..layers.linear import ReplicatedLinear
from ..layers.logits_processor import LogitsProcessor
from ..parallel import state as ps
from .llama import DenseMLP
from .mimo_v2_flash import MiMoV2Attention


class MiMoV2NextNLayer(nn.Module):
    def __init__(self, config, layer_id: int, dtype):
        super().__init__()
        H = config.hidden_size
        eps = getattr(config, "layernorm_epsilon", None) or getattr(config, "rms_norm_eps", 1e-6)
        self.enorm = RMSNorm(H, eps, dtype)
        self.hnorm = RMSNorm(H, eps, dtype)
        self.eh_proj = ReplicatedLinear(2 * H, H, False, dtype)
        self.input_layernorm = RMSNorm(H, eps, dtype)
        self.self_attn = MiMoV2Attention(config, layer_id, dtype, swa=True)
        self.pre_mlp_layernorm = RMSNorm(H, eps, dtype)
        self.mlp = DenseMLP(H, config.intermediate_size, dtype)
        self.final_layernorm = RMSNorm(H, eps, dtype)

    def forward(self, emb, hidden, fb):
        x = self.eh_proj(torch.cat([self.enorm(emb), self.hnorm(hidden)], dim=-1))
        x = x + self.self_attn(self.input_layernorm(x), fb)
        x = x + self.mlp(self.pre_mlp_layernorm(x))
        return self.final_layernorm(x)


class _Holder(nn.Module):
    pass


class MiMoV2NextN(nn.Module):
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
        self.num_mtp_layers = self.num_kv_layers = n
        tp = ps.tp_size()
        # the draft cache holds the sliding-window head layout, not the full-attention one
        self.kv_shape = (max(1, config.swa_num_key_value_heads // tp), config.swa_head_dim)
        self.model = _Holder()
        self.model.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        self.model.mtp = _Holder()
        self.model.mtp.layers = nn.ModuleList([MiMoV2NextNLayer(config, j, dtype) for j in range(n)])
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.logits_processor = LogitsProcessor(config.vocab_size)

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
        layers = self.model.mtp.layers
        if getattr(si, "mtp_all_layers", False):
            h = [layer(emb, hidden, forward_batch) for layer in layers][0]
        else:
            h = layers[min(int(getattr(si, "mtp_layer", 0) or 0), self.num_mtp_layers - 1)](emb, hidden, forward_batch)
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
            if ".mtp.layers." not in name:
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
        return loaded | {"model.embed_tokens.weight", "lm_head.weight"}


class MiMoV2MTPForCausalLM(MiMoV2NextN):
    """Name under which the reference registers the MiMo-V2 MTP draft model (`models/mimo_v2_nextn.py`)."""


EntryClass = [MiMoV2NextN, MiMoV2MTPForCausalLM]
