"""Gemma 2: alternating sliding-window / global attention, attention-logit and final-logit
soft-capping, GeGLU MLP, `(1 + w)` RMSNorm before and after both sub-blocks, embeddings
scaled by sqrt(hidden) (reference `python/sgl_jax/srt/models/gemma2.py`)."""

from __future__ import annotations

import torch
from torch import nn

from ..layers.activation import GeluAndMul
from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding, get_rope
from ..layers.layernorm import GemmaRMSNorm
from ..layers.linear import MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear
from ..layers.logits_processor import LogitsProcessor
from ..layers.radix_attention import RadixAttention
from .llama import LlamaForCausalLM


class Gemma2Attention(nn.Module):
    def __init__(self, config, layer_id, dtype, sliding_window):
        super().__init__()
        H = config.hidden_size
        self.head_dim = config.head_dim
        self.qkv_proj = QKVParallelLinear(H, self.head_dim, config.num_attention_heads, config.num_key_value_heads,
                                          getattr(config, "attention_bias", False), dtype)
        self.o_proj = RowParallelLinear(config.num_attention_heads * self.head_dim, H,
                                        getattr(config, "attention_bias", False), dtype)
        self.rotary_emb = get_rope(self.head_dim, self.head_dim, config.max_position_embeddings,
                                   getattr(config, "rope_theta", 10000.0), True, None, dtype)
        self.attn = RadixAttention(self.qkv_proj.num_heads, self.head_dim,
                                   float(config.query_pre_attn_scalar) ** -0.5, self.qkv_proj.num_kv_heads, layer_id,
                                   sliding_window, getattr(config, "attn_logit_softcapping", None) or 0.0)

    def forward(self, x, forward_batch):
        return self.o_proj(self.attn(self.qkv_proj(x), forward_batch, self.rotary_emb))


class Gemma2MLP(nn.Module):
    def __init__(self, config, dtype):
        super().__init__()
        self.gate_up_proj = MergedColumnParallelLinear(config.hidden_size, [config.intermediate_size] * 2, False, dtype)
        self.down_proj = RowParallelLinear(config.intermediate_size, config.hidden_size, False, dtype)
        self.act_fn = GeluAndMul("tanh")

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_up_proj(x)))


class Gemma2DecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype):
        super().__init__()
        eps = config.rms_norm_eps
        H = config.hidden_size
        types = getattr(config, "layer_types", None)
        is_sliding = (types[layer_id] == "sliding_attention") if types else (layer_id % 2 == 0)
        self.is_sliding = is_sliding
        self.self_attn = Gemma2Attention(config, layer_id, dtype, config.sliding_window if is_sliding else 0)
        self.mlp = Gemma2MLP(config, dtype)
        self.input_layernorm = GemmaRMSNorm(H, eps, dtype)
        self.post_attention_layernorm = GemmaRMSNorm(H, eps, dtype)
        self.pre_feedforward_layernorm = GemmaRMSNorm(H, eps, dtype)
        self.post_feedforward_layernorm = GemmaRMSNorm(H, eps, dtype)

    def forward(self, x, forward_batch):
        h = self.self_attn(self.input_layernorm(x), forward_batch)
        x = x + self.post_attention_layernorm(h)
        h = self.mlp(self.pre_feedforward_layernorm(x))
        return x + self.post_feedforward_layernorm(h)


class Gemma2Model(nn.Module):
    def __init__(self, config, dtype):
        super().__init__()
        self.config = config
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        self.layers = nn.ModuleList([Gemma2DecoderLayer(config, i, dtype) for i in range(config.num_hidden_layers)])
        self.norm = GemmaRMSNorm(config.hidden_size, config.rms_norm_eps, dtype)
        self.normalizer = float(config.hidden_size) ** 0.5

    def forward(self, input_ids, forward_batch, input_embeds=None):
        x = self.embed_tokens(input_ids) if input_embeds is None else input_embeds
        x = x * torch.tensor(self.normalizer, dtype=x.dtype)
        for layer in self.layers:
            x = layer(x, forward_batch)
        return self.norm(x)


class Gemma2ForCausalLM(LlamaForCausalLM):
    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        self.config = config
        self.dtype = dtype
        self.model = Gemma2Model(config, dtype)
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = True
        self.logits_processor = LogitsProcessor(config.vocab_size, getattr(config, "final_logit_softcapping", None))
        self.capture_aux_hidden_states = False
        self.swa_layer_ids = [i for i, l in enumerate(self.model.layers) if l.is_sliding]

    def forward(self, input_ids, forward_batch, input_embeds=None):
        return self.logits_processor(self.model(input_ids, forward_batch, input_embeds), self.lm_head, forward_batch)


EntryClass = [Gemma2ForCausalLM]
