"""MiMo-V2-Flash / MiMo-V2-Pro (reference `python/sgl_jax/srt/models/mimo_v2_flash.py`,
`mimo_v2_pro.py`): layers follow `hybrid_layer_pattern` — sliding-window layers with their own
head count / head sizes and a learned attention-sink bias, full-attention layers otherwise; the
value head may be narrower than the key head (it is zero-padded inside the KV cache); FFNs follow
`moe_layer_freq` (sigmoid routing with correction bias, no shared expert)."""

from __future__ import annotations

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding, get_rope
from ..layers.layernorm import RMSNorm
from ..layers.linear import QKVParallelLinear, RowParallelLinear
from ..layers.logits_processor import LogitsProcessor
from ..layers.radix_attention import RadixAttention
from ..parallel import state as ps
from .deepseek_v3 import DeepseekMoE
from .llama import DenseMLP, LlamaForCausalLM
from .moe_loading import load_sparse_weights


def _is_swa(config, i: int) -> bool:
    pat = getattr(config, "hybrid_layer_pattern", None)
    return bool(pat is not None and 0 <= i < len(pat) and pat[i] == 1)


def _is_moe(config, i: int) -> bool:
    f = getattr(config, "moe_layer_freq", None)
    return bool(f is not None and not isinstance(f, int) and 0 <= i < len(f) and f[i])


class MiMoV2Attention(nn.Module):
    def __init__(self, config, layer_id, dtype, swa: bool):
        super().__init__()
        H = config.hidden_size
        if swa:
            nh, nkv = config.swa_num_attention_heads, config.swa_num_key_value_heads
            hd, vd = config.swa_head_dim, getattr(config, "swa_v_head_dim", None) or config.swa_head_dim
            theta = getattr(config, "swa_rope_theta", None) or getattr(config, "rope_theta", 1e6)
            window = getattr(config, "sliding_window_size", None) or getattr(config, "sliding_window", 0) or 0
            sink = bool(getattr(config, "add_swa_attention_sink_bias", False))
        else:
            nh, nkv = config.num_attention_heads, config.num_key_value_heads
            hd, vd = config.head_dim, getattr(config, "v_head_dim", None) or config.head_dim
            theta = getattr(config, "rope_theta", 1e6)
            window = 0
            sink = bool(getattr(config, "add_full_attention_sink_bias", False))
        self.hd, self.vd = hd, vd
        self.qkv_proj = QKVParallelLinear(H, hd, nh, nkv, getattr(config, "attention_bias", False), dtype, v_head_dim=vd)
        self.o_proj = RowParallelLinear(nh * vd, H, False, dtype)
        prf = getattr(config, "partial_rotary_factor", 1.0)
        self.rotary_emb = get_rope(hd, int(hd * prf), config.max_position_embeddings, theta, True,
                                   getattr(config, "rope_scaling", None), dtype)
        self.value_scale = getattr(config, "attention_value_scale", None)
        self.attn = RadixAttention(self.qkv_proj.num_heads, hd, hd ** -0.5, self.qkv_proj.num_kv_heads, layer_id, window)
        self.attention_sink_bias = nn.Parameter(torch.zeros(self.qkv_proj.num_heads, dtype=torch.float32),
                                                requires_grad=False) if sink else None
        self._sink_rank = self.qkv_proj.tp_rank

    def weight_loader(self, param, w, shard_id=None):      # the sink bias is sharded with the query heads
        n = param.shape[0]
        param.data.copy_(w.float().narrow(0, self._sink_rank * n, n))

    def forward(self, x, fb):
        qp = self.qkv_proj
        qkv = qp(x)
        if self.vd != self.hd or self.value_scale is not None:
            q, k, v = qkv.split([qp.q_size, qp.k_size, qp.v_size], dim=-1)
            if self.value_scale is not None:
                v = v * self.value_scale
            if self.vd != self.hd:       # the cache stores V at key width
                v = torch.nn.functional.pad(v.view(-1, qp.num_kv_heads, self.vd), (0, self.hd - self.vd)).flatten(1)
            qkv = torch.cat([q, k, v], dim=-1)
        o = self.attn(qkv, fb, self.rotary_emb, sinks=self.attention_sink_bias)
        if self.vd != self.hd:
            o = o.view(-1, qp.num_heads, self.hd)[..., : self.vd].reshape(-1, qp.num_heads * self.vd)
        return self.o_proj(o)


class MiMoV2DecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype):
        super().__init__()
        self.is_swa = _is_swa(config, layer_id)
        self.self_attn = MiMoV2Attention(config, layer_id, dtype, self.is_swa)
        self.is_sparse = _is_moe(config, layer_id)
        self.mlp = DeepseekMoE(config, layer_id, dtype) if self.is_sparse else \
            DenseMLP(config.hidden_size, config.intermediate_size, dtype)
        eps = getattr(config, "layernorm_epsilon", None) or getattr(config, "rms_norm_eps", 1e-6)
        self.input_layernorm = RMSNorm(config.hidden_size, eps, dtype)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps, dtype)

    def forward(self, x, fb):
        x = x + self.self_attn(self.input_layernorm(x), fb)
        h = self.post_attention_layernorm(x)
        if self.is_sparse:
            y = self.mlp.partial(h)
            if self.mlp.tp_size > 1:
                y = ps.all_reduce(y)
        else:
            y = self.mlp(h)
        return x + y


class MiMoV2FlashForCausalLM(LlamaForCausalLM):
    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        if not hasattr(config, "n_routed_experts"):
            config.n_routed_experts = getattr(config, "num_experts", 0)
        if not hasattr(config, "n_shared_experts"):
            config.n_shared_experts = 0
        self.config, self.dtype = config, dtype
        model = nn.Module()
        model.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        model.layers = nn.ModuleList([MiMoV2DecoderLayer(config, i, dtype) for i in range(config.num_hidden_layers)])
        eps = getattr(config, "layernorm_epsilon", None) or getattr(config, "rms_norm_eps", 1e-6)
        model.norm = RMSNorm(config.hidden_size, eps, dtype)
        self.model = model
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        self.logits_processor = LogitsProcessor(config.vocab_size)
        self.capture_aux_hidden_states = False
        swa = [i for i in range(config.num_hidden_layers) if _is_swa(config, i)]
        if swa and len(swa) < config.num_hidden_layers:
            self.swa_layer_ids = swa
            tp = ps.tp_size()
            self.swa_kv_shape = (max(1, config.swa_num_key_value_heads // tp), config.swa_head_dim)

    def forward(self, input_ids, fb, input_embeds=None):
        x = self.model.embed_tokens(input_ids) if input_embeds is None else input_embeds
        for layer in self.model.layers:
            x = layer(x, fb)
        return self.logits_processor(self.model.norm(x), self.lm_head, fb)

    def load_weights(self, weights):
        loaded = load_sparse_weights(self, weights, max_layer=self.config.num_hidden_layers, skip=("mtp.",))
        return loaded


class MiMoV2ProForCausalLM(MiMoV2FlashForCausalLM):
    pass


EntryClass = [MiMoV2FlashForCausalLM, MiMoV2ProForCausalLM]
