"""Qwen3-Omni thinker: audio encoder, vision encoder and the mixture-of-experts language model."""
