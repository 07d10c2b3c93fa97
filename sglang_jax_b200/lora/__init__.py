"""Multi-adapter LoRA serving (reference `python/sgl_jax/srt/lora/`): adapters are loaded
into stacked device buffers, each request names an adapter, and one batched
gather-matmul (BGMV) adds every token's own low-rank update to the base projection."""
