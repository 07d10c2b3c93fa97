"""Ling-linear / Ring-linear (reference `python/sgl_jax/srt/models/bailing_moe_linear.py`): groups of
Lightning linear-attention layers closed by one softmax-attention layer, over the Ling MoE FFN."""

from __future__ import annotations

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding
from ..layers.layernorm import RMSNorm
from ..layers.linear_attention import LightningAttention
from ..layers.logits_processor import LogitsProcessor
from ..parallel import state as ps
from .bailing_moe import BailingMoeV2ForCausalLM
from .deepseek_v3 import DeepseekMoE
from .llama import DenseAttention, DenseMLP, LlamaForCausalLM
from .moe_loading import STACKED, load_sparse_weights


def _is_linear(config, layer_id: int) -> bool:
    g = getattr(config, "layer_group_size", 1) or 1
    return g > 1 and (layer_id + 1) % g != 0


class BailingLinearLayer(nn.Module):
    def __init__(self, config, layer_id, dtype, kv_layer_id, linear_index):
        super().__init__()
        self.is_linear = _is_linear(config, layer_id)
        if self.is_linear:
            self.attention = LightningAttention(config, linear_index, layer_id, dtype)
        else:
            self.self_attn = DenseAttention(config, kv_layer_id, dtype, qkv_bias=getattr(config, "use_qkv_bias", False),
                                            o_bias=getattr(config, "use_bias", False),
                                            qk_norm=getattr(config, "use_qk_norm", False))
        self.is_sparse = layer_id >= getattr(config, "first_k_dense_replace", 0) and config.n_routed_experts > 0
        self.mlp = DeepseekMoE(config, layer_id, dtype, correction_bias=True) if self.is_sparse else \
            DenseMLP(config.hidden_size, config.intermediate_size, dtype)
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype)

    def forward(self, x, fb):
        h = self.input_layernorm(x)
        h = self.attention(h, fb) if self.is_linear else self.self_attn.o_proj(self.self_attn(h, fb))
        x = x + h
        h = self.post_attention_layernorm(x)
        if self.is_sparse:
            y = self.mlp.partial(h)
            if self.mlp.tp_size > 1:
                y = ps.all_reduce(y)
        else:
            y = self.mlp(h)
        return x + y


class BailingMoeLinearForCausalLM(LlamaForCausalLM):
    is_hybrid_linear = True
    _renames = BailingMoeV2ForCausalLM._renames + [(".attention.g_norm.weight", ".attention.g_norm")]

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        config.n_routed_experts = getattr(config, "num_experts", 0)
        config.n_shared_experts = getattr(config, "num_shared_experts", 0) or 0
        config.scoring_func = getattr(config, "score_function", "sigmoid")
        for k, v in (("norm_topk_prob", True), ("n_group", 0), ("topk_group", 0)):
            if not hasattr(config, k):
                setattr(config, k, v)
        if not getattr(config, "head_dim", None):
            config.head_dim = config.hidden_size // config.num_attention_heads
        self.use_bias = bool(getattr(config, "moe_router_enable_expert_bias", False))
        self.config, self.dtype = config, dtype
        config.layer_types = ["linear_attention" if _is_linear(config, i) else "full_attention"
                              for i in range(config.num_hidden_layers)]
        model = nn.Module()
        model.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        layers, kv_id, lin_id = [], 0, 0
        for i in range(config.num_hidden_layers):
            layers.append(BailingLinearLayer(config, i, dtype, kv_id, lin_id))
            if _is_linear(config, i):
                lin_id += 1
            else:
                kv_id += 1
        model.layers = nn.ModuleList(layers)
        model.norm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype)
        self.model = model
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        self.logits_processor = LogitsProcessor(config.vocab_size)
        self.capture_aux_hidden_states = False
        self.num_kv_layers = max(kv_id, 1)
        self.recurrent_spec = dict(num_layers=max(lin_id, 1), conv_dim=1, conv_kernel=2,
                                   num_heads=config.num_attention_heads, head_k_dim=config.head_dim,
                                   head_v_dim=config.head_dim)

    def forward(self, input_ids, fb, input_embeds=None):
        x = self.model.embed_tokens(input_ids) if input_embeds is None else input_embeds
        for layer in self.model.layers:
            x = layer(x, fb)
        return self.logits_processor(self.model.norm(x), self.lm_head, fb)

    def load_weights(self, weights):
        lin = {i for i in range(self.config.num_hidden_layers) if _is_linear(self.config, i)}

        def routed():
            # softmax layers use the fused-qkv renames of Ling; linear layers keep `attention.*` names
            for name, w in weights:
                if name.startswith("model.layers.") and int(name.split(".")[2]) in lin:
                    name = name.replace(".attention.g_norm.weight", ".attention.g_norm")
                    name = name.replace(".mlp.gate.expert_bias", ".mlp.gate.e_score_correction_bias")
                    yield name, w
                else:
                    for a, b in BailingMoeV2ForCausalLM._renames:
                        name = name.replace(a, b)
                    yield name, w

        loaded = load_sparse_weights(self, routed(), max_layer=self.config.num_hidden_layers,
                                     stacked=[s for s in STACKED if s[0] != ".qkv_proj"])
        if not self.use_bias:
            loaded |= {n for n, _ in self.named_parameters() if n.endswith("e_score_correction_bias")}
        return loaded


class BailingMoeV2_5ForCausalLM(BailingMoeLinearForCausalLM):
    """The architecture string Ling-2.5 / Ring-2.5 linear-attention checkpoints carry (reference
    `models/bailing_moe_linear.py` `EntryClass`)."""


EntryClass = [BailingMoeLinearForCausalLM, BailingMoeV2_5ForCausalLM]
