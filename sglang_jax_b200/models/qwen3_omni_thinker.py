"""Language half of the Qwen3-Omni thinker and of Qwen3-VL-MoE (reference
`python/sgl_jax/srt/multimodal/models/qwen3_omni_moe/qwen3_omni_thinker.py`): a Qwen3-MoE decoder
with interleaved three-stream rotary positions; merged vision features of intermediate encoder
layers are added to the residual stream after the first decoder layers (deep-stack).  Audio /
image / video embeddings, positions and deep-stack features arrive per request as `mm_inputs`."""

from __future__ import annotations

import torch

from .qwen3_moe import Qwen3MoeForCausalLM


def _text_config(config):
    tc = getattr(config, "text_config", None)
    if tc is None and getattr(config, "thinker_config", None) is not None:
        tc = getattr(config.thinker_config, "text_config", None)
    tc = tc or config
    rp = getattr(tc, "rope_parameters", None) or getattr(tc, "rope_scaling", None) or {}
    sec = list(rp.get("mrope_section") or [24, 20, 20])
    if rp.get("rope_theta") and not getattr(tc, "rope_theta", None):
        tc.rope_theta = rp["rope_theta"]
    tc.rope_scaling = {"rope_type": "default", "mrope_section": sec,
                       "mrope_interleaved": bool(rp.get("mrope_interleaved", True))}
    tc.rope_parameters = None
    if not hasattr(tc, "tie_word_embeddings"):
        tc.tie_word_embeddings = bool(getattr(config, "tie_word_embeddings", False))
    if getattr(tc, "num_experts", None) is None and getattr(tc, "num_local_experts", None):
        tc.num_experts = tc.num_local_experts          # configs re-saved by recent `transformers` use this name
    return tc


class Qwen3OmniMoeThinkerForConditionalGeneration(Qwen3MoeForCausalLM):
    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__(_text_config(config), dtype, quant_config)

    def load_weights(self, weights):
        def text_only():
            for n, w in weights:
                if any(t in n for t in ("audio_tower.", "visual.", "talker.", "code2wav.", "code_predictor.")):
                    continue
                n = n.replace("thinker.", "", 1) if n.startswith("thinker.") else n
                yield n.replace("model.language_model.", "model."), w
        return super().load_weights(text_only())


class Qwen3OmniMoeForConditionalGeneration(Qwen3OmniMoeThinkerForConditionalGeneration):
    pass


class Qwen3VLMoeForConditionalGeneration(Qwen3OmniMoeThinkerForConditionalGeneration):
    pass


EntryClass = [Qwen3OmniMoeThinkerForConditionalGeneration, Qwen3OmniMoeForConditionalGeneration,
              Qwen3VLMoeForConditionalGeneration]
