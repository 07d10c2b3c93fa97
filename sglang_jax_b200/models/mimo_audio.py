"""Main transformer of MiMo-Audio (reference
`python/sgl_jax/srt/multimodal/models/mimo_audio/mimo_audio_backbone.py`: `MiMoAudioForCausalLM`):
a Qwen2 decoder that steps over groups of audio frames.  Group embeddings come in as input
embeddings; the local patch encoder / decoder around it live in
`multimodal/models/mimo_audio_backbone.py`."""

from __future__ import annotations

from .qwen2 import Qwen2ForCausalLM

_LOCAL = ("local_transformer", "input_local_transformer", "speech_embeddings", "local_transformer_lm_heads",
          "speech_group_downcast", "hidden_states_downcast")


class MiMoAudioForCausalLM(Qwen2ForCausalLM):
    def load_weights(self, weights):
        return super().load_weights((n, w) for n, w in weights if not n.startswith(_LOCAL))


EntryClass = [MiMoAudioForCausalLM]
