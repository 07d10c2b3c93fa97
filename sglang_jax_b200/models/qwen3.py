"""Qwen3 dense decoder: Llama blocks + per-head RMSNorm on q and k before RoPE, no biases
(reference `python/sgl_jax/srt/models/qwen3.py:28-610`)."""

from .llama import LlamaForCausalLM


class Qwen3ForCausalLM(LlamaForCausalLM):
    def _attn_kw(self, config):
        return dict(qkv_bias=getattr(config, "attention_bias", False), o_bias=False, qk_norm=True)


EntryClass = Qwen3ForCausalLM
