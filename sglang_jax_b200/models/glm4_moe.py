"""GLM-4.5 / GLM-4.6 MoE (reference `python/sgl_jax/srt/models/glm4_moe.py`): GQA attention with
biased q/k/v, optional per-head q/k RMSNorm, half-rotary RoPE; the first `first_k_dense_replace`
layers are dense, the rest route with sigmoid scores + correction bias over expert groups and
add shared experts."""

from __future__ import annotations

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead
from ..layers.fused_block import partial_add_norm, row_linear_add_norm
from ..layers.layernorm import RMSNorm
from ..layers.logits_processor import LogitsProcessor
from .deepseek_v3 import DeepseekMoE
from .llama import DenseAttention, DenseMLP, DenseModel, LlamaForCausalLM
from .moe_loading import load_sparse_weights


class Glm4MoeDecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype, **attn_kw):
        super().__init__()
        eps = config.rms_norm_eps
        self.self_attn = DenseAttention(config, layer_id, dtype, **attn_kw)
        self.is_sparse = layer_id >= getattr(config, "first_k_dense_replace", 0) and \
            getattr(config, "n_routed_experts", 0) > 0
        self.mlp = DeepseekMoE(config, layer_id, dtype, correction_bias=True) if self.is_sparse else \
            DenseMLP(config.hidden_size, config.intermediate_size, dtype)
        self.input_layernorm = RMSNorm(config.hidden_size, eps, dtype)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps, dtype)

    def forward(self, h_normed, residual, fb, next_norm):
        a = self.self_attn(h_normed, fb)
        h, residual = row_linear_add_norm(self.self_attn.o_proj, a, residual, self.post_attention_layernorm)
        if self.is_sparse:
            return partial_add_norm(lambda out: self.mlp.partial(h, out), h.shape[0], h.shape[1], residual, next_norm,
                                    self.mlp.tp_size, block=self.mlp, x=h)
        act = self.mlp.act_fn(self.mlp.gate_up_proj(h))
        return row_linear_add_norm(self.mlp.down_proj, act, residual, next_norm)


class Glm4MoeModel(DenseModel):
    layer_cls = Glm4MoeDecoderLayer


class Glm4MoeForCausalLM(LlamaForCausalLM):
    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        if not hasattr(config, "scoring_func"):
            config.scoring_func = "sigmoid"
        self.config = config
        self.dtype = dtype
        self.model = Glm4MoeModel(config, dtype, **self._attn_kw(config))
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        self.logits_processor = LogitsProcessor(config.vocab_size)
        self.capture_aux_hidden_states = False

    def _attn_kw(self, config):
        return dict(qkv_bias=getattr(config, "attention_bias", False), o_bias=False,
                    qk_norm=getattr(config, "use_qk_norm", False))

    def load_weights(self, weights):
        # layers past `num_hidden_layers` are the multi-token-prediction head
        return load_sparse_weights(self, weights, max_layer=self.config.num_hidden_layers)


EntryClass = [Glm4MoeForCausalLM]
