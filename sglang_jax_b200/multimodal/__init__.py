"""Multimodal serving: a pipeline of stages (text/vision/audio encoders, diffusion transformer,
VAE, language backbone), each with its own scheduler, executor and GPUs, orchestrated by a
global scheduler (reference `python/sgl_jax/srt/multimodal/`, `docs/architecture/12-multimodal.md`)."""
