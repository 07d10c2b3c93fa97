"""Speculative decoding: draft heads propose a token tree, the target verifies it in one
forward (reference `python/sgl_jax/srt/speculative/`)."""
