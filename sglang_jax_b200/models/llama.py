"""Llama-family dense decoders: Llama 2/3, Mistral, InternLM3, Phi-3 (fused qkv / gate_up
checkpoints), and the shared building blocks that Qwen2/Qwen3 reuse.

Parameter names are the HF ones (`model.layers.{i}.self_attn.q_proj.weight`, ...), as in
the reference (`python/sgl_jax/srt/models/llama.py`, weight map of
`python/sgl_jax/srt/models/qwen3.py:421-539`); q/k/v and gate/up are stacked into one
fused GEMM each at load time.
"""

from __future__ import annotations

from typing import Iterable

import torch
from torch import nn

from ..layers.activation import SiluAndMul
from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding, get_rope
from ..layers.fused_block import row_linear_add_norm
from ..layers.layernorm import RMSNorm
from ..layers.linear import MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear
from ..layers.logits_processor import LogitsProcessor
from ..layers.radix_attention import RadixAttention
from ..utils.precision_tracer import precision_tracer


class DenseMLP(nn.Module):
    def __init__(self, hidden_size, intermediate_size, dtype, bias=False):
        super().__init__()
        self.gate_up_proj = MergedColumnParallelLinear(hidden_size, [intermediate_size] * 2, bias, dtype)
        self.down_proj = RowParallelLinear(intermediate_size, hidden_size, bias, dtype, reduce_results=True)
        self.act_fn = SiluAndMul()

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_up_proj(x)))


class DenseAttention(nn.Module):
    def __init__(self, config, layer_id: int, dtype, qkv_bias=False, o_bias=False, qk_norm=False,
                 sliding_window=0):
        super().__init__()
        hidden = config.hidden_size
        self.total_heads = config.num_attention_heads
        self.total_kv_heads = getattr(config, "num_key_value_heads", None) or self.total_heads
        self.head_dim = getattr(config, "head_dim", None) or hidden // self.total_heads
        self.qkv_proj = QKVParallelLinear(hidden, self.head_dim, self.total_heads, self.total_kv_heads,
                                          qkv_bias, dtype)
        self.o_proj = RowParallelLinear(self.total_heads * self.head_dim, hidden, o_bias, dtype)
        eps = getattr(config, "rms_norm_eps", 1e-6)
        self.q_norm = RMSNorm(self.head_dim, eps, dtype) if qk_norm else None
        self.k_norm = RMSNorm(self.head_dim, eps, dtype) if qk_norm else None
        rope_theta = getattr(config, "rope_theta", None)
        rope_scaling = getattr(config, "rope_scaling", None)
        rp = getattr(config, "rope_parameters", None)
        if isinstance(rp, dict):
            rope_theta = rope_theta or rp.get("rope_theta")
            if rp.get("rope_type", "default") != "default":
                rope_scaling = rope_scaling or rp
        self.rotary_emb = get_rope(self.head_dim, self.head_dim,
                                   getattr(config, "max_position_embeddings", 8192),
                                   rope_theta or 10000.0, True, rope_scaling, dtype,
                                   getattr(config, "partial_rotary_factor", 1.0))
        self.attn = RadixAttention(self.qkv_proj.num_heads, self.head_dim, self.head_dim ** -0.5,
                                   self.qkv_proj.num_kv_heads, layer_id, sliding_window)

    def forward(self, hidden_states, forward_batch):
        qkv = self.qkv_proj(hidden_states)
        return self.attn(qkv, forward_batch, self.rotary_emb, self.q_norm, self.k_norm)


class DenseDecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype, **attn_kw):
        super().__init__()
        eps = getattr(config, "rms_norm_eps", 1e-6)
        self.self_attn = DenseAttention(config, layer_id, dtype, **attn_kw)
        self.mlp = DenseMLP(config.hidden_size, config.intermediate_size, dtype,
                            getattr(config, "mlp_bias", False))
        self.input_layernorm = RMSNorm(config.hidden_size, eps, dtype)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps, dtype)

    def forward(self, hidden_normed, residual, forward_batch, next_norm, next_consumer=None):
        """`hidden_normed` is this layer's already-normalised input; returns the next layer's
        normalised input and the updated residual stream.  `next_consumer`: the projection of the next layer
        that reads the returned activations first (its GEMM then absorbs the all-gather wait)."""
        attn_out = self.self_attn(hidden_normed, forward_batch)
        h, residual = row_linear_add_norm(self.self_attn.o_proj, attn_out, residual,
                                          self.post_attention_layernorm, consumer=self.mlp.gate_up_proj)
        act = self.mlp.act_fn(self.mlp.gate_up_proj(h))
        return row_linear_add_norm(self.mlp.down_proj, act, residual, next_norm, consumer=next_consumer)


class DenseModel(nn.Module):
    layer_cls = DenseDecoderLayer

    def __init__(self, config, dtype, **attn_kw):
        super().__init__()
        self.config = config
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        self.layers = nn.ModuleList([self.layer_cls(config, i, dtype, **attn_kw)
                                     for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, getattr(config, "rms_norm_eps", 1e-6), dtype)
        self.layers_to_capture: list[int] = []
        # layers of this class read their input only through `self_attn.qkv_proj`, so the previous layer may
        # leave the all-gather wait to that GEMM; subclasses with other first readers switch this off
        self.defer_gather = self.layer_cls is DenseDecoderLayer

    def forward(self, input_ids, forward_batch, input_embeds=None):
        residual = self.embed_tokens(input_ids) if input_embeds is None else input_embeds
        h = self.layers[0].input_layernorm(residual)
        aux = []
        n = len(self.layers)
        tracing = precision_tracer.enabled
        if tracing:
            precision_tracer.begin_forward()
            precision_tracer.record(residual, "embed_tokens", forward_batch.forward_mode.name)
        for i, layer in enumerate(self.layers):
            if i in self.layers_to_capture:
                # the fused add-norm kernels update `residual` in place: keep a copy, not a reference
                aux.append(residual.clone())
            nxt = self.layers[i + 1].input_layernorm if i + 1 < n else self.norm
            if self.defer_gather and i + 1 < n:
                h, residual = layer(h, residual, forward_batch, nxt, self.layers[i + 1].self_attn.qkv_proj)
            else:
                h, residual = layer(h, residual, forward_batch, nxt)
            deep = forward_batch.extras.get("deepstack")
            if deep is not None and i < deep.shape[0]:
                # vision features join the residual stream after the first layers (deep-stack)
                residual = residual + deep[i].to(residual.dtype)
                h = nxt(residual)
            if tracing:
                precision_tracer.record(residual, "layer_residual", forward_batch.forward_mode.name, i)
                precision_tracer.record(h, "layer_output_normed", forward_batch.forward_mode.name, i)
        return (h, aux) if self.layers_to_capture else h


class LlamaForCausalLM(nn.Module):
    """Base causal LM.  Subclasses set the attention flavour through `attn_kw`."""

    attn_kw: dict = {}
    # (param fragment in this model, fragment in the checkpoint, shard id)
    stacked_params_mapping = [
        (".qkv_proj", ".q_proj", "q"), (".qkv_proj", ".k_proj", "k"), (".qkv_proj", ".v_proj", "v"),
        (".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1),
    ]

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        self.config = config
        self.dtype = dtype
        self.model = DenseModel(config, dtype, **self._attn_kw(config))
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        self.logits_processor = LogitsProcessor(config.vocab_size,
                                                getattr(config, "final_logit_softcapping", None))
        self.capture_aux_hidden_states = False

    def _attn_kw(self, config) -> dict:
        return dict(qkv_bias=getattr(config, "attention_bias", False),
                    o_bias=getattr(config, "attention_bias", False))

    def forward(self, input_ids, forward_batch, input_embeds=None):
        hidden = self.model(input_ids, forward_batch, input_embeds)
        aux = None
        if isinstance(hidden, tuple):
            hidden, aux = hidden
        out = self.logits_processor(hidden, self.lm_head, forward_batch)
        if aux is not None:
            out.extras["aux_hidden_states"] = aux
        return out

    def get_embed_and_head(self):
        return self.model.embed_tokens.weight, self.lm_head.weight

    def set_eagle3_layers_to_capture(self, layer_ids=None):
        n = self.config.num_hidden_layers
        self.model.layers_to_capture = layer_ids or [2, n // 2, n - 3]
        self.capture_aux_hidden_states = True

    # ------------------------------------------------------------------ loading
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        modules = dict(self.named_modules())
        loaded = set()
        for name, w in weights:
            if "rotary_emb.inv_freq" in name or "rotary_emb.cos_cached" in name:
                continue
            if name == "lm_head.weight" and self.tie:
                continue
            if name.startswith("model.vision_tower") or name.startswith("visual."):
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
        self.post_load_weights()
        return loaded

    def post_load_weights(self):
        if self.tie:
            self.lm_head.tie_to(self.model.embed_tokens)


class MistralForCausalLM(LlamaForCausalLM):
    pass


class InternLM3ForCausalLM(LlamaForCausalLM):
    def _attn_kw(self, config):
        return dict(qkv_bias=getattr(config, "qkv_bias", False), o_bias=getattr(config, "bias", False))


class Phi3ForCausalLM(LlamaForCausalLM):
    """Phi-3 checkpoints already store fused `qkv_proj` / `gate_up_proj` tensors."""
    stacked_params_mapping = []


EntryClass = [LlamaForCausalLM, MistralForCausalLM, InternLM3ForCausalLM, Phi3ForCausalLM]
