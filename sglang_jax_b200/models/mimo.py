"""MiMo-7B: a Qwen2-style dense decoder that ships extra multi-token-prediction (MTP)
layers in the same checkpoint (reference `python/sgl_jax/srt/models/mimo.py`).  The main
model ignores the `model.mtp_layers.*` weights; `mimo_mtp.MiMoMTP` loads only those."""

from .qwen2 import Qwen2ForCausalLM


class MiMoForCausalLM(Qwen2ForCausalLM):
    def load_weights(self, weights):
        return super().load_weights((n, w) for n, w in weights if "mtp_layers" not in n)


EntryClass = [MiMoForCausalLM]
