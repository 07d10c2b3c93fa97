"""Host-memory tier of the KV cache (HiCache L2) and the staging pool used by prefill/decode
disaggregation.

Reference: `python/sgl_jax/srt/mem_cache/host_kv_pool.py` (`LRUHostKVPool` :266,
`QueueHostKVPool` :110).  The reference stages device pages through jitted gathers and
blocking transfers driven from a thread pool.  Here every layer has a pinned host mirror
`[host_pages, page_elems]`; a page moves with one launch of the page-copy kernel per layer,
which reads/writes the pinned memory directly over the host link, so a backup or a
load-back is a handful of asynchronous launches on a side stream and an event.
"""

from __future__ import annotations

import logging
from collections import deque

import numpy as np
import torch

logger = logging.getLogger(__name__)


def _layer_views(device_pool) -> list[torch.Tensor]:
    """Every KV layer buffer of a device pool as a 2-D `[pages, page_elems]` view."""
    bufs = []
    inner = getattr(device_pool, "inner", device_pool)
    pools = [inner.full_pool, inner.swa_pool] if hasattr(inner, "full_pool") else [inner]
    for p in pools:
        for b in p.kv_buffer:
            bufs.append(b.view(b.shape[0], -1))
    return bufs


class HostKVPool:
    """Pinned host pages mirroring the layout of a device pool, with a page free list."""

    def __init__(self, device_pool, num_pages: int, pin_memory: bool | None = None):
        self.device_pool = device_pool
        self.page_size = device_pool.page_size
        self.dev_views = _layer_views(device_pool)
        self.layer_num = len(self.dev_views)
        self.num_pages = int(num_pages)
        on_gpu = self.dev_views[0].is_cuda
        pin = on_gpu if pin_memory is None else pin_memory
        self.host_views = [torch.empty((self.num_pages, v.shape[1]), dtype=v.dtype, pin_memory=pin)
                           for v in self.dev_views]
        self.free_pages = deque(range(self.num_pages))
        self.on_gpu = on_gpu

    # ------------------------------------------------------------------ accounting
    def available_pages(self) -> int:
        return len(self.free_pages)

    def size_bytes(self) -> int:
        return sum(v.numel() * v.element_size() for v in self.host_views)

    def alloc(self, n: int) -> np.ndarray | None:
        if n > len(self.free_pages):
            return None
        return np.asarray([self.free_pages.popleft() for _ in range(n)], dtype=np.int64)

    def free(self, pages) -> None:
        self.free_pages.extend(int(p) for p in np.asarray(pages).ravel())

    # ------------------------------------------------------------------ movement
    def backup_from_device(self, device_pages: np.ndarray, host_pages: np.ndarray) -> None:
        """device -> host, asynchronous on the current stream when the pool is on a GPU."""
        self._move(self.host_views, self.dev_views, host_pages, device_pages)

    def load_to_device(self, host_pages: np.ndarray, device_pages: np.ndarray) -> None:
        self._move(self.dev_views, self.host_views, device_pages, host_pages)

    def _move(self, dst_views, src_views, dst_pages, src_pages):
        n = len(dst_pages)
        if n == 0:
            return
        if self.on_gpu:
            from ..ops import native
            dev = self.dev_views[0].device
            d = torch.as_tensor(np.asarray(dst_pages, np.int64)).to(dev, non_blocking=True)
            s = torch.as_tensor(np.asarray(src_pages, np.int64)).to(dev, non_blocking=True)
            for dv, sv in zip(dst_views, src_views):
                native.kv_page_copy(dv, sv, d, s)
        else:
            d = torch.as_tensor(np.asarray(dst_pages, np.int64))
            s = torch.as_tensor(np.asarray(src_pages, np.int64))
            for dv, sv in zip(dst_views, src_views):
                dv[d] = sv[s]


class LRUHostKVPool(HostKVPool):
    """The HiCache tier: the radix tree decides what lives here and evicts by LRU."""


class QueueHostKVPool(HostKVPool):
    """FIFO staging area for KV pages in flight between a prefill and a decode engine:
    `put` reserves pages and copies them out of the device pool, `get` loads the oldest
    entry back into device pages and releases it."""

    def __init__(self, device_pool, num_pages: int, pin_memory: bool | None = None):
        super().__init__(device_pool, num_pages, pin_memory)
        self.entries: "deque[tuple[str, np.ndarray]]" = deque()

    def put(self, key: str, device_pages: np.ndarray) -> bool:
        pages = self.alloc(len(device_pages))
        if pages is None:
            return False
        self.backup_from_device(np.asarray(device_pages, np.int64), pages)
        self.entries.append((key, pages))
        return True

    # -- reservations: the PD transfer threads stage pages here (reserve -> copy -> send / scatter -> release)
    def reserve(self, n: int, timeout: float = 30.0) -> np.ndarray | None:
        """`n` staging pages, waiting up to `timeout` seconds for other transfers to release theirs; `None` when the
        pool is smaller than `n` or the wait ran out (the caller then stages through a one-off buffer)."""
        import threading
        import time
        if not hasattr(self, "_cv"):
            self._cv = threading.Condition()
        if n > self.num_pages:
            return None
        deadline = time.monotonic() + timeout
        with self._cv:
            while len(self.free_pages) < n:
                left = deadline - time.monotonic()
                if left <= 0:
                    return None
                self._cv.wait(left)
            return self.alloc(n)

    def release(self, pages) -> None:
        import threading
        if not hasattr(self, "_cv"):
            self._cv = threading.Condition()
        with self._cv:
            self.free(pages)
            self._cv.notify_all()

    def host_bytes(self, layer: int, host_pages: np.ndarray) -> bytes:
        """The staged pages of one layer as one contiguous byte string (page order = `host_pages` order)."""
        v = self.host_views[layer][torch.as_tensor(np.asarray(host_pages, np.int64))]
        return v.contiguous().view(torch.uint8).numpy().tobytes()

    def fill_host(self, layer: int, host_pages: np.ndarray, raw) -> None:
        v = self.host_views[layer]
        src = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(v.dtype).view(len(host_pages), v.shape[1])
        v[torch.as_tensor(np.asarray(host_pages, np.int64))] = src

    def get(self, key: str, device_pages: np.ndarray) -> bool:
        for i, (k, pages) in enumerate(self.entries):
            if k == key:
                if len(pages) != len(device_pages):
                    raise ValueError("page count mismatch")
                self.load_to_device(pages, np.asarray(device_pages, np.int64))
                del self.entries[i]
                self.free(pages)
                return True
        return False
