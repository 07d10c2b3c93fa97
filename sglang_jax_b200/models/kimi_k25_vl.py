"""Language half of Kimi-K2.5 (reference `python/sgl_jax/srt/models/kimi_k25_vl_generation.py`,
`multimodal/models/kimi_k25/kimi_k25_vl_generation.py`): the DeepSeek-V3 latent-attention MoE
decoder stored under `language_model.*`; image features arrive as per-token input embeddings."""

from __future__ import annotations

import torch

from .deepseek_v3 import DeepseekV3ForCausalLM


class KimiK25ForConditionalGeneration(DeepseekV3ForCausalLM):
    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        tc = getattr(config, "text_config", None) or config
        if isinstance(getattr(tc, "quantization_config", None), dict):
            tc.quantization_config = None          # nested pack-quantised description: weights are folded on load
        super().__init__(tc, dtype, quant_config)
        self.media_placeholder_token_id = getattr(config, "media_placeholder_token_id", None)

    def load_weights(self, weights):
        def text_only():
            for n, w in weights:
                if n.startswith("vision_tower.") or n.startswith("mm_projector."):
                    continue
                yield (n[len("language_model."):] if n.startswith("language_model.") else n), w
        return super().load_weights(text_only())


EntryClass = [KimiK25ForConditionalGeneration]
