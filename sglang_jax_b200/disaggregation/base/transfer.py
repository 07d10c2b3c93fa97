"""What a data-plane backend has to provide (reference
`python/sgl_jax/srt/disaggregation/base/transfer.py:139`)."""

from __future__ import annotations

import dataclasses
from typing import Protocol

import numpy as np


def chunk_transfer_id(transfer_id: str, chunk: int) -> str:
    """Chunked prefill registers one transfer per chunk under a derived id."""
    return f"{transfer_id}#c{chunk}"


@dataclasses.dataclass
class KVLayout:
    """Shape facts both ends must agree on before bytes are copied page for page."""
    page_size: int
    num_layers: int
    page_bytes_per_layer: list[int]
    dtype: str
    tp_size: int = 1
    tp_rank: int = 0

    def compatible(self, other: "KVLayout") -> str | None:
        for f in ("page_size", "num_layers", "page_bytes_per_layer", "dtype", "tp_size"):
            if getattr(self, f) != getattr(other, f):
                return f"KV layout mismatch on {f}: {getattr(self, f)} != {getattr(other, f)}"
        return None


class TransferBackend(Protocol):
    name: str

    def start(self) -> str:
        """Bring the endpoint up; returns the address peers use to reach it."""

    def register(self, transfer_id: str, pages: np.ndarray, meta: dict) -> None:
        """Prefill: make `pages` of the local pool pullable under `transfer_id`."""

    def unregister(self, transfer_id: str) -> None: ...

    def pull(self, addr: str, transfer_id: str, dst_pages: np.ndarray) -> dict:
        """Decode: copy the registered pages into `dst_pages` of the local pool; returns the
        sender's `meta` (first token, ...).  Blocking; raises on failure or timeout."""

    def stop(self) -> None: ...
