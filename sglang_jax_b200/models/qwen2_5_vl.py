"""Language half of Qwen2.5-VL (reference
`python/sgl_jax/srt/multimodal/models/qwen2_5VL/qwen2_5_vl_generation.py`): a Qwen2 decoder whose
rotary embedding is driven by three position streams (`mrope_section` lanes each for the temporal,
height and width index).  Image / video embeddings arrive from the vision stage as per-token
input embeddings together with the 3-D positions; text-only requests behave like Qwen2."""

from __future__ import annotations

import torch

from .qwen2 import Qwen2ForCausalLM


def _text_config(config):
    tc = getattr(config, "text_config", None) or config
    sec = None
    for src in (getattr(tc, "rope_scaling", None), getattr(tc, "rope_parameters", None),
                getattr(config, "rope_scaling", None)):
        if isinstance(src, dict) and src.get("mrope_section"):
            sec = list(src["mrope_section"])
            if src.get("rope_theta") and not getattr(tc, "rope_theta", None):
                tc.rope_theta = src["rope_theta"]
            break
    if sec:
        tc.rope_scaling = {"rope_type": "default", "mrope_section": sec}
        tc.rope_parameters = None
    for k in ("vocab_size", "tie_word_embeddings"):
        if not hasattr(tc, k) and hasattr(config, k):
            setattr(tc, k, getattr(config, k))
    return tc


class Qwen2_5_VLForConditionalGeneration(Qwen2ForCausalLM):
    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__(_text_config(config), dtype, quant_config)
        self.image_token_id = getattr(config, "image_token_id", None)
        self.video_token_id = getattr(config, "video_token_id", None)

    def load_weights(self, weights):
        def text_only():
            for n, w in weights:
                if ".visual." in n or n.startswith("visual."):
                    continue
                yield n.replace("model.language_model.", "model."), w
        return super().load_weights(text_only())


class Qwen2VLForConditionalGeneration(Qwen2_5_VLForConditionalGeneration):
    pass


EntryClass = [Qwen2_5_VLForConditionalGeneration, Qwen2VLForConditionalGeneration]
