"""Kimi-Linear (reference `python/sgl_jax/srt/models/kimi_linear.py`): a hybrid of Kimi Delta
Attention layers (recurrent state, no KV cache) and position-free MLA layers (latent KV cache),
with a dense first layer and sigmoid-routed MoE FFNs with shared experts."""

from __future__ import annotations

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding
from ..layers.layernorm import RMSNorm
from ..layers.linear_attention import KimiDeltaAttention
from ..layers.logits_processor import LogitsProcessor
from ..parallel import state as ps
from .deepseek_v3 import DeepseekMoE, MLAAttention
from .llama import DenseMLP, LlamaForCausalLM
from .moe_loading import load_sparse_weights


def _kda_layers(config) -> set[int]:
    lc = config.linear_attn_config
    # checkpoint lists are 1-based
    return {i - 1 for i in lc.get("kda_layers", [])}


class KimiDecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype, kv_layer_id, linear_index):
        super().__init__()
        self.is_kda = layer_id in _kda_layers(config)
        if self.is_kda:
            self.self_attn = KimiDeltaAttention(config, linear_index, dtype)
        else:
            self.self_attn = MLAAttention(config, kv_layer_id, dtype)
            self.self_attn.skip_rope = bool(getattr(config, "mla_use_nope", True))
        first_dense = getattr(config, "first_k_dense_replace", 0)
        freq = getattr(config, "moe_layer_freq", 1) or 1
        n_exp = getattr(config, "n_routed_experts", 0) or 0
        self.is_sparse = n_exp > 0 and layer_id >= first_dense and layer_id % freq == 0
        self.mlp = DeepseekMoE(config, layer_id, dtype, correction_bias=True) if self.is_sparse else \
            DenseMLP(config.hidden_size, config.intermediate_size, dtype)
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype)

    def forward(self, x, fb):
        h = self.self_attn(self.input_layernorm(x), fb)
        if not self.is_kda:
            h = self.self_attn.o_proj(h)
        x = x + h
        h = self.post_attention_layernorm(x)
        if self.is_sparse:
            y = self.mlp.partial(h)
            if self.mlp.tp_size > 1:
                y = ps.all_reduce(y)
        else:
            y = self.mlp(h)
        return x + y


class KimiLinearForCausalLM(LlamaForCausalLM):
    is_hybrid_linear = True

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        config = getattr(config, "text_config", None) or config
        for a, b in (("n_routed_experts", "num_experts"), ("n_shared_experts", "num_shared_experts"),
                     ("num_experts_per_tok", "num_experts_per_token"), ("scoring_func", "moe_router_activation_func")):
            if not hasattr(config, a) and hasattr(config, b):
                setattr(config, a, getattr(config, b))
        if not hasattr(config, "norm_topk_prob"):
            config.norm_topk_prob = bool(getattr(config, "moe_renormalize", True))
        self.config = config
        self.dtype = dtype
        kda = _kda_layers(config)
        config.layer_types = ["linear_attention" if i in kda else "full_attention"
                              for i in range(config.num_hidden_layers)]
        model = nn.Module()
        model.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        layers, kv_id, lin_id = [], 0, 0
        for i in range(config.num_hidden_layers):
            layers.append(KimiDecoderLayer(config, i, dtype, kv_id, lin_id))
            if i in kda:
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
        lc = config.linear_attn_config
        self.recurrent_spec = dict(num_layers=max(lin_id, 1), conv_dim=3 * lc["num_heads"] * lc["head_dim"],
                                   conv_kernel=lc["short_conv_kernel_size"], num_heads=lc["num_heads"],
                                   head_k_dim=lc["head_dim"], head_v_dim=lc["head_dim"])

    def forward(self, input_ids, fb, input_embeds=None):
        x = self.model.embed_tokens(input_ids) if input_embeds is None else input_embeds
        for layer in self.model.layers:
            x = layer(x, fb)
        return self.logits_processor(self.model.norm(x), self.lm_head, fb)

    def post_load_weights(self):
        super().post_load_weights()
        for layer in self.model.layers:
            if not layer.is_kda:
                layer.self_attn.absorb()

    def load_weights(self, weights):
        ren = [(".block_sparse_moe.", ".mlp."), (".self_attn.q_conv1d.weight", ".self_attn.q_conv1d_weight"),
               (".self_attn.k_conv1d.weight", ".self_attn.k_conv1d_weight"),
               (".self_attn.v_conv1d.weight", ".self_attn.v_conv1d_weight"),
               (".mlp.gate.e_score_correction_bias", ".mlp.gate.e_score_correction_bias")]
        stacked = [(".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1)]
        return load_sparse_weights(self, weights, renames=ren, stacked=stacked,
                                   expert_proj={"w1": "gate", "w3": "up", "w2": "down", "gate_proj": "gate",
                                                "up_proj": "up", "down_proj": "down"})


EntryClass = [KimiLinearForCausalLM]
