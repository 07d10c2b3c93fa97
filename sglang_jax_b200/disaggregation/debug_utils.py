"""KV digests for checking that a transfer delivered the bytes it was given (reference
`python/sgl_jax/srt/disaggregation/debug_utils.py`)."""

from __future__ import annotations

import hashlib

import numpy as np
import torch


def kv_digest(device_pool, pages) -> str:
    """SHA-256 over the bytes of `pages` in every layer, in layer order."""
    from ..mem_cache.host_kv_pool import _layer_views
    idx = torch.as_tensor(np.asarray(pages, np.int64))
    h = hashlib.sha256()
    for v in _layer_views(device_pool):
        h.update(v[idx.to(v.device)].contiguous().view(torch.uint8).cpu().numpy().tobytes())
    return h.hexdigest()
