"""Ling / Bailing MoE (v1 and v2; reference `python/sgl_jax/srt/models/bailing_moe.py`).
Architecturally a GLM-4-MoE-style decoder — GQA attention with optional per-head q/k norm and
partial rotary, dense first layers, then sigmoid/softmax routed experts over groups with an
optional expert bias, plus shared experts — stored under its own parameter names
(`word_embeddings`, `attention.query_key_value`, `attention.dense`, `mlp.gate.expert_bias`)."""

from __future__ import annotations

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead
from ..layers.logits_processor import LogitsProcessor
from .glm4_moe import Glm4MoeModel
from .llama import LlamaForCausalLM
from .moe_loading import STACKED, load_sparse_weights


class BailingMoeV2ForCausalLM(LlamaForCausalLM):
    _renames = [("model.word_embeddings.", "model.embed_tokens."), (".attention.query_key_value.", ".self_attn.qkv_proj."),
                (".attention.dense.", ".self_attn.o_proj."), (".attention.query_layernorm.", ".self_attn.q_norm."),
                (".attention.key_layernorm.", ".self_attn.k_norm."),
                (".mlp.gate.expert_bias", ".mlp.gate.e_score_correction_bias")]

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        # express the config in the vocabulary the shared sparse block reads
        config.n_routed_experts = getattr(config, "num_experts", 0)
        config.n_shared_experts = getattr(config, "num_shared_experts", 0) or 0
        config.scoring_func = getattr(config, "score_function", "softmax")
        if not hasattr(config, "norm_topk_prob"):
            config.norm_topk_prob = True
        if not hasattr(config, "n_group"):
            config.n_group, config.topk_group = 0, 0
        if not hasattr(config, "head_dim") or config.head_dim is None:
            config.head_dim = config.hidden_size // config.num_attention_heads
        self.use_bias = bool(getattr(config, "moe_router_enable_expert_bias", False))
        self.config = config
        self.dtype = dtype
        self.model = Glm4MoeModel(config, dtype, qkv_bias=getattr(config, "use_qkv_bias", False),
                                  o_bias=getattr(config, "use_bias", False), qk_norm=getattr(config, "use_qk_norm", False))
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        self.logits_processor = LogitsProcessor(config.vocab_size)
        self.capture_aux_hidden_states = False

    def load_weights(self, weights):
        loaded = load_sparse_weights(self, weights, renames=self._renames, max_layer=self.config.num_hidden_layers,
                                     stacked=[s for s in STACKED if s[0] != ".qkv_proj"])
        if not self.use_bias:
            # no expert bias in this checkpoint: the selection bias stays zero
            loaded |= {n for n, _ in self.named_parameters() if n.endswith("e_score_correction_bias")}
        return loaded


class BailingMoeForCausalLM(BailingMoeV2ForCausalLM):
    pass


class BailingMoEForCausalLM(BailingMoeV2ForCausalLM):
    pass


EntryClass = [BailingMoeV2ForCausalLM, BailingMoeForCausalLM, BailingMoEForCausalLM]
