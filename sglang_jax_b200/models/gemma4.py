"""Gemma 4 text model (reference `python/sgl_jax/srt/models/gemma4.py`).

Sliding-window layers use `head_dim` / `num_key_value_heads` and plain RoPE; global layers use
`global_head_dim`, proportional RoPE over a fraction of the head and — with `attention_k_eq_v`
— `num_global_key_value_heads` heads whose values are the (un-rotated, scale-free-normed) key
projection.  q/k get a weighted per-head RMSNorm, v a scale-free one; attention logits are not
scaled.  Every sub-block is wrapped in pre- and post-norms; with `enable_moe_block` a routed
GeGLU expert block (router on the scale-free-normed residual, per-expert output scales) runs
beside the dense MLP.  The layer output is multiplied by a learned per-layer scalar.
"""

from __future__ import annotations

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding, get_rope
from ..layers.gate import GateLogit, TopK
from ..layers.layernorm import RMSNorm
from ..layers.linear import QKVParallelLinear, RowParallelLinear
from ..layers.logits_processor import LogitsProcessor
from ..layers.moe import FusedMoE
from ..layers.radix_attention import RadixAttention
from ..parallel import state as ps
from .gemma2 import Gemma2MLP
from .llama import LlamaForCausalLM
from .moe_loading import load_sparse_weights


def _layer_type(config, i):
    t = getattr(config, "layer_types", None)
    return t[i] if t and i < len(t) else "full_attention"


def _attn_shape(config, sliding: bool):
    """(kv heads, head dim, values-are-keys) of a layer kind.  Accepts both the checkpoint's names
    (`global_head_dim`, `num_global_key_value_heads`) and the `swa_*` aliases."""
    nh = config.num_attention_heads
    base_hd = getattr(config, "head_dim", None) or config.hidden_size // nh
    base_kv = getattr(config, "num_key_value_heads", nh)
    if sliding:
        return getattr(config, "swa_num_key_value_heads", None) or base_kv, \
            getattr(config, "swa_head_dim", None) or base_hd, False
    k_eq_v = bool(getattr(config, "attention_k_eq_v", False))
    hd = getattr(config, "global_head_dim", None) or base_hd
    kv = (getattr(config, "num_global_key_value_heads", None) or base_kv) if k_eq_v else base_kv
    return kv, hd, k_eq_v


def _scale_free_norm(x, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


class Gemma4Attention(nn.Module):
    def __init__(self, config, layer_id, dtype):
        super().__init__()
        kind = _layer_type(config, layer_id)
        self.is_sliding = kind == "sliding_attention"
        nkv, hd, self.k_eq_v = _attn_shape(config, self.is_sliding)
        self.head_dim, self.eps = hd, getattr(config, "rms_norm_eps", 1e-6)
        bias = getattr(config, "attention_bias", False)
        self.qkv_proj = QKVParallelLinear(config.hidden_size, hd, config.num_attention_heads, nkv, bias, dtype)
        self.o_proj = RowParallelLinear(config.num_attention_heads * hd, config.hidden_size, bias, dtype)
        self.q_norm = RMSNorm(hd, self.eps, dtype)
        self.k_norm = RMSNorm(hd, self.eps, dtype)
        rp = dict((getattr(config, "rope_parameters", None) or {}).get(kind, {}))
        if self.is_sliding:
            theta = rp.get("rope_theta", getattr(config, "rope_local_base_freq", 10000.0))
            self.rotary_emb = get_rope(hd, hd, config.max_position_embeddings, theta, True, None, dtype,
                                       rp.get("partial_rotary_factor", 1.0))
        else:
            theta = rp.get("rope_theta", getattr(config, "rope_theta", 1000000.0))
            prop = rp.get("rope_type", "proportional") == "proportional"
            self.rotary_emb = get_rope(hd, hd, config.max_position_embeddings, theta, True,
                                       {"proportional": True} if prop else None, dtype,
                                       rp.get("partial_rotary_factor", 0.25 if prop else 1.0))
        self.attn = RadixAttention(self.qkv_proj.num_heads, hd, 1.0, self.qkv_proj.num_kv_heads, layer_id,
                                   config.sliding_window if self.is_sliding else 0)

    def forward(self, x, fb):
        qp = self.qkv_proj
        qkv = qp(x)
        q, k, v = qkv.split([qp.q_size, qp.k_size, qp.v_size], dim=-1)
        v = _scale_free_norm(v.reshape(-1, qp.num_kv_heads, self.head_dim), self.eps).flatten(1)
        o = self.attn(torch.cat([q, k, v], dim=-1), fb, self.rotary_emb, self.q_norm, self.k_norm)
        return self.o_proj(o)


class Gemma4Router(nn.Module):
    def __init__(self, config, dtype):
        super().__init__()
        H, E = config.hidden_size, config.num_experts
        self.eps = getattr(config, "rms_norm_eps", 1e-6)
        self.root = H ** -0.5
        self.scale = nn.Parameter(torch.ones(H, dtype=dtype), requires_grad=False)
        self.per_expert_scale = nn.Parameter(torch.ones(E, dtype=dtype), requires_grad=False)
        self.proj = GateLogit(H, E, dtype)

    def weight_loader(self, param, w, shard_id=None):
        param.data.copy_(w)

    def forward(self, x):
        return self.proj(_scale_free_norm(x, self.eps) * self.scale * self.root)


class Gemma4DecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype):
        super().__init__()
        H, eps = config.hidden_size, getattr(config, "rms_norm_eps", 1e-6)
        self.self_attn = Gemma4Attention(config, layer_id, dtype)
        self.is_sliding = self.self_attn.is_sliding
        self.mlp = Gemma2MLP(config, dtype)
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                  "post_feedforward_layernorm"):
            setattr(self, n, RMSNorm(H, eps, dtype))
        self.layer_scalar = nn.Parameter(torch.ones(1, dtype=dtype), requires_grad=False)
        self.enable_moe_block = bool(getattr(config, "enable_moe_block", False))
        if self.enable_moe_block:
            k = getattr(config, "num_experts_per_tok", None) or getattr(config, "top_k_experts", 8)
            self.router = Gemma4Router(config, dtype)
            self.topk = TopK(k, renormalize=True)
            self.experts = FusedMoE(config.num_experts, H,
                                    getattr(config, "moe_intermediate_size", None) or config.intermediate_size,
                                    dtype, layer_id=layer_id, activation="gelu")
            for n in ("post_feedforward_layernorm_1", "post_feedforward_layernorm_2", "pre_feedforward_layernorm_2"):
                setattr(self, n, RMSNorm(H, eps, dtype))

    def weight_loader(self, param, w, shard_id=None):
        param.data.copy_(w.reshape(param.shape))

    def forward(self, x, fb):
        x = x + self.post_attention_layernorm(self.self_attn(self.input_layernorm(x), fb))
        h = self.mlp(self.pre_feedforward_layernorm(x))
        if self.enable_moe_block:
            h1 = self.post_feedforward_layernorm_1(h)
            w, ids = self.topk(self.router(x))
            w = w * self.router.per_expert_scale.float()[ids.long()]
            h2 = self.experts(self.pre_feedforward_layernorm_2(x), w, ids)
            if self.experts.tp_size > 1:
                h2 = ps.all_reduce(h2)
            h = h1 + self.post_feedforward_layernorm_2(h2)
        x = x + self.post_feedforward_layernorm(h)
        return x * self.layer_scalar


class Gemma4ForCausalLM(LlamaForCausalLM):
    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        config = getattr(config, "text_config", config)
        if getattr(config, "hidden_size_per_layer_input", 0) or getattr(config, "num_kv_shared_layers", 0):
            raise NotImplementedError("Gemma-4 per-layer input embeddings / shared-KV layers (the E2B/E4B variants) "
                                      "are not supported")
        self.config, self.dtype = config, dtype
        model = nn.Module()
        model.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        model.layers = nn.ModuleList([Gemma4DecoderLayer(config, i, dtype) for i in range(config.num_hidden_layers)])
        model.norm = RMSNorm(config.hidden_size, getattr(config, "rms_norm_eps", 1e-6), dtype)
        self.model = model
        self.normalizer = float(config.hidden_size) ** 0.5
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", True))
        self.logits_processor = LogitsProcessor(config.vocab_size, getattr(config, "final_logit_softcapping", None))
        self.capture_aux_hidden_states = False
        swa = [i for i, l in enumerate(model.layers) if l.is_sliding]
        if swa and len(swa) < config.num_hidden_layers:
            self.swa_layer_ids = swa
            a = model.layers[swa[0]].self_attn
            self.swa_kv_shape = (a.qkv_proj.num_kv_heads, a.head_dim)
            full = next(l for l in model.layers if not l.is_sliding).self_attn
            self.full_kv_shape = (full.qkv_proj.num_kv_heads, full.head_dim)

    def forward(self, input_ids, fb, input_embeds=None):
        if input_embeds is None:
            x = self.model.embed_tokens(input_ids)
            x = x * torch.tensor(self.normalizer, dtype=x.dtype)
        else:
            x = input_embeds
        for layer in self.model.layers:
            x = layer(x, fb)
        return self.logits_processor(self.model.norm(x), self.lm_head, fb)

    def load_weights(self, weights):
        def stream():
            for name, w in weights:
                if "vision_tower" in name or "audio_tower" in name or "embed_vision" in name or "embed_audio" in name:
                    continue
                name = name.replace("model.language_model.", "model.").replace("language_model.model.", "model.")
                yield name, w
                if ".self_attn.k_proj." in name:
                    i = int(name.split(".")[2])
                    if self.model.layers[i].self_attn.k_eq_v:      # values are the key projection
                        yield name.replace(".k_proj.", ".v_proj."), w
        return load_sparse_weights(self, stream())


class Gemma4ForConditionalGeneration(Gemma4ForCausalLM):
    pass


EntryClass = [Gemma4ForCausalLM, Gemma4ForConditionalGeneration]
