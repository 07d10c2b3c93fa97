"""Qwen / Qwen2 / Qwen2.5 dense decoders: Llama blocks with biased q/k/v projections
(reference `python/sgl_jax/srt/models/qwen2.py`, `qwen.py`)."""

from .llama import LlamaForCausalLM


class Qwen2ForCausalLM(LlamaForCausalLM):
    def _attn_kw(self, config):
        return dict(qkv_bias=True, o_bias=False)


class QWenLMHeadModel(Qwen2ForCausalLM):
    """First-generation Qwen: same math; the checkpoint uses `transformer.h.*` names which
    are rewritten on load."""

    _rename = [("transformer.h.", "model.layers."), ("transformer.wte.", "model.embed_tokens."),
               ("transformer.ln_f.", "model.norm."), (".ln_1.", ".input_layernorm."),
               (".ln_2.", ".post_attention_layernorm."), (".attn.c_attn.", ".self_attn.qkv_proj."),
               (".attn.c_proj.", ".self_attn.o_proj."), (".mlp.w2.", ".mlp.gate_proj."),
               (".mlp.w1.", ".mlp.up_proj."), (".mlp.c_proj.", ".mlp.down_proj.")]

    def load_weights(self, weights):
        def renamed():
            for n, w in weights:
                for a, b in self._rename:
                    n = n.replace(a, b)
                yield n, w
        return super().load_weights(renamed())


EntryClass = [Qwen2ForCausalLM, QWenLMHeadModel]
