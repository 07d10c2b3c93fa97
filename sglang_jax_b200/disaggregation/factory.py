"""Construction of the KV transfer backend an engine uses (reference
`python/sgl_jax/srt/disaggregation/factory.py: create_transfer_backend`, which chooses between the
`jax.experimental.transfer` backend and the optional native Raiden extension and sizes the latter's staging pool).

Two data paths exist here behind one control channel (`transfer/zmq_transfer.py`):

* `tcp`: pages are staged through pinned host memory and travel as message frames (any topology, CPU too);
* `cuda_ipc`: the decode engine maps the prefill engine's KV buffers through CUDA IPC and its page-copy kernel reads
  them over NVLink (both engines in one NVLink domain).  `--disaggregation-use-raiden`, the reference's switch for
  its native device-to-device path, selects this one.
"""

from __future__ import annotations

import logging

logger = logging.getLogger(__name__)

_ALIASES = {"tcp": "tcp", "zmq": "tcp", "host": "tcp", "cuda_ipc": "cuda_ipc", "nvlink": "cuda_ipc"}


def pick_transfer_mode(server_args, on_gpu: bool) -> str:
    """`--disaggregation-enable-d2h` (or a pool that is not on a GPU) forces the host-staged path."""
    if not on_gpu or server_args.disaggregation_enable_d2h:
        return "tcp"
    if getattr(server_args, "disaggregation_use_raiden", False):
        return "cuda_ipc"
    name = getattr(server_args, "disaggregation_transfer_backend", None) or "tcp"
    if name not in _ALIASES:
        raise ValueError(f"unknown KV transfer backend {name!r} (tcp | cuda_ipc)")
    return _ALIASES[name]


def staging_pages(server_args, max_req_input_len: int, page_size: int) -> int:
    """Pages of pinned staging one transfer may need on the host-staged path: a whole prompt, or one prefill chunk
    when chunked hand-over is enabled (the reference sizes its Raiden slots the same way, `factory.py:21-44`)."""
    tokens = int(max_req_input_len)
    if server_args.disaggregation_enable_chunk_prefill_transfer:
        chunk = server_args.chunked_prefill_size
        if not chunk or chunk <= 0:
            raise ValueError("chunk transfer requires a positive chunked_prefill_size")
        tokens = min(tokens, int(chunk))
    if server_args.disaggregation_d2h_max_tokens:
        tokens = min(tokens, int(server_args.disaggregation_d2h_max_tokens))
    return max(1, (tokens + page_size - 1) // page_size)


def create_transfer_backend(device_pool, server_args, *, local_host: str, role: str, shared_secret: str | None,
                            max_req_input_len: int | None = None):
    from ..mem_cache.host_kv_pool import _layer_views
    from .transfer.zmq_transfer import ZmqTransferBackend
    on_gpu = _layer_views(device_pool)[0].is_cuda
    mode = pick_transfer_mode(server_args, on_gpu)
    port = server_args.disaggregation_transfer_port if role == "prefill" else 0
    staging = 0
    if mode == "tcp" and on_gpu:
        # pinned staging: `--disaggregation-d2h-pool-size` transfers of one prompt (or one chunk) each, capped at 4 GiB
        views = _layer_views(device_pool)
        page_bytes = sum(int(v.shape[1] * v.element_size()) for v in views)
        per = staging_pages(server_args, max_req_input_len or server_args.context_length or 8192, device_pool.page_size)
        staging = max(per, min(per * max(1, server_args.disaggregation_d2h_pool_size), (4 << 30) // max(page_bytes, 1)))
    backend = ZmqTransferBackend(device_pool, local_host, port, mode, shared_secret,
                                 server_args.disaggregation_pull_timeout_seconds, staging_pages=staging)
    logger.info("PD %s engine: KV transfer backend %s", role, mode)
    return backend
