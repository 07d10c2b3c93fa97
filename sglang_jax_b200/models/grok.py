"""Grok-1 / Grok-2 (reference `python/sgl_jax/srt/models/grok.py`): four norms per layer
(pre/post attention, pre/post MoE), attention-logit soft-capping, GELU experts routed by a
soft-capped router with softmax over all experts and un-renormalised top-k weights, optional
dense MLP in parallel with the experts (`residual_moe`, outputs averaged by 1/sqrt(2)),
embedding and output multipliers."""

from __future__ import annotations

import math

import torch
from torch import nn

from ..layers.activation import GeluAndMul
from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding, get_rope
from ..layers.layernorm import RMSNorm
from ..layers.linear import MergedColumnParallelLinear, QKVParallelLinear, ReplicatedLinear, RowParallelLinear
from ..layers.logits_processor import LogitsProcessor
from ..layers.moe import FusedMoE
from ..layers.radix_attention import RadixAttention
from ..parallel import state as ps
from .llama import LlamaForCausalLM
from .moe_loading import load_sparse_weights


class Grok1MLP(nn.Module):
    def __init__(self, hidden, inter, dtype):
        super().__init__()
        self.gate_up_proj = MergedColumnParallelLinear(hidden, [inter] * 2, False, dtype)
        self.down_proj = RowParallelLinear(inter, hidden, False, dtype, reduce_results=False)
        self.act_fn = GeluAndMul("tanh")

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_up_proj(x)))


class Grok1MoE(nn.Module):
    def __init__(self, config, layer_id, dtype):
        super().__init__()
        E = config.num_local_experts
        self.top_k = config.num_experts_per_tok
        self.gate = ReplicatedLinear(config.hidden_size, E, False, torch.float32)
        self.softcap = float(getattr(config, "router_logit_softcapping", 30.0) or 0.0)
        inter = getattr(config, "moe_intermediate_size", None) or config.intermediate_size
        self.experts = FusedMoE(E, config.hidden_size, inter, dtype, layer_id=layer_id, activation="gelu")

    def forward(self, x):
        logits = torch.nn.functional.linear(x.float(), self.gate.weight.float())
        if self.softcap:
            logits = torch.tanh(logits / self.softcap) * self.softcap
        probs = torch.softmax(logits, dim=-1)
        w, ids = torch.topk(probs, self.top_k, dim=-1)
        return self.experts(x, w, ids.to(torch.int32))        # partial sum (not yet reduced)


class Grok1Attention(nn.Module):
    def __init__(self, config, layer_id, dtype):
        super().__init__()
        H = config.hidden_size
        self.head_dim = getattr(config, "head_dim", None) or H // config.num_attention_heads
        self.qkv_proj = QKVParallelLinear(H, self.head_dim, config.num_attention_heads, config.num_key_value_heads,
                                          getattr(config, "attention_bias", False), dtype)
        self.o_proj = RowParallelLinear(config.num_attention_heads * self.head_dim, H, False, dtype)
        rotary_dim = self.head_dim // 2 if getattr(config, "rope_rotate_half_dims", False) else self.head_dim
        self.rotary_emb = get_rope(self.head_dim, rotary_dim, config.max_position_embeddings,
                                   getattr(config, "rope_theta", 10000), True, getattr(config, "rope_scaling", None), dtype)
        cap = max(float(getattr(config, "attn_logit_softcapping", 30.0) or 0.0), 0.0)
        scale = getattr(config, "attn_scale", None) or self.head_dim ** -0.5
        self.attn = RadixAttention(self.qkv_proj.num_heads, self.head_dim, scale, self.qkv_proj.num_kv_heads,
                                   layer_id, 0, cap)

    def forward(self, x, fb):
        return self.o_proj(self.attn(self.qkv_proj(x), fb, self.rotary_emb))


class Grok1DecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype):
        super().__init__()
        eps = config.rms_norm_eps
        H = config.hidden_size
        self.self_attn = Grok1Attention(config, layer_id, dtype)
        self.block_sparse_moe = Grok1MoE(config, layer_id, dtype)
        self.residual_moe = bool(getattr(config, "residual_moe", False))
        self.mlp = Grok1MLP(H, config.intermediate_size, dtype) if self.residual_moe else None
        self.pre_attn_norm = RMSNorm(H, eps, dtype)
        self.post_attn_norm = RMSNorm(H, eps, dtype)
        self.pre_moe_norm = RMSNorm(H, eps, dtype)
        self.post_moe_norm = RMSNorm(H, eps, dtype)

    def forward(self, x, fb):
        x = x + self.post_attn_norm(self.self_attn(self.pre_attn_norm(x), fb))
        h = self.pre_moe_norm(x)
        y = self.block_sparse_moe(h)
        if self.mlp is not None:
            y = (y.float() + self.mlp(h).float()).to(y.dtype)
        if ps.tp_size() > 1:
            y = ps.all_reduce(y)
        if self.mlp is not None:
            y = y * torch.tensor(1.0 / math.sqrt(2.0), dtype=y.dtype)
        return x + self.post_moe_norm(y)


class Grok1Model(nn.Module):
    def __init__(self, config, dtype):
        super().__init__()
        self.config = config
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        self.layers = nn.ModuleList([Grok1DecoderLayer(config, i, dtype) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype)

    def forward(self, input_ids, fb, input_embeds=None):
        x = self.embed_tokens(input_ids) if input_embeds is None else input_embeds
        mult = getattr(self.config, "embedding_multiplier_scale", None)
        if mult:
            x = x * torch.tensor(float(mult), dtype=x.dtype)
        for layer in self.layers:
            x = layer(x, fb)
        return self.norm(x)


class Grok1ForCausalLM(LlamaForCausalLM):
    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        self.config = config
        self.dtype = dtype
        self.model = Grok1Model(config, dtype)
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        self.logits_processor = LogitsProcessor(config.vocab_size, getattr(config, "final_logit_softcapping", None))
        self.output_multiplier = float(getattr(config, "output_multiplier_scale", 1.0) or 1.0)
        self.capture_aux_hidden_states = False

    def forward(self, input_ids, fb, input_embeds=None):
        h = self.model(input_ids, fb, input_embeds)
        if self.output_multiplier != 1.0:
            # the multiplier scales the logits; folding it into the hidden state is the same linear map
            h = h * torch.tensor(self.output_multiplier, dtype=h.dtype)
        return self.logits_processor(h, self.lm_head, fb)

    def load_weights(self, weights):
        return load_sparse_weights(self, weights, expert_proj={"w1": "gate", "w3": "up", "w2": "down"})


EntryClass = [Grok1ForCausalLM]
