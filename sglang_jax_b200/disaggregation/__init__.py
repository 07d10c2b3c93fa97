"""Prefill/decode disaggregation: a prefill engine builds the KV cache of a prompt, a decode
engine pulls it and generates (reference `python/sgl_jax/srt/disaggregation/`).

Control plane: HTTP bootstrap registry + heartbeats, a router that pairs a prefill and a
decode endpoint per request, an acknowledgement side channel and a timeout reaper.
Data plane (`transfer/`): page-granular KV pulls — over CUDA IPC peer memory with the
page-copy kernel when both engines sit on one NVLink domain, through pinned host staging
and TCP otherwise."""
