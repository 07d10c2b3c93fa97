"""Moves KV pages between the device pool and the host tier without blocking the scheduler.

Reference: `python/sgl_jax/srt/mem_cache/hicache_controller.py` (thread pool + ack queues,
because its transfers block).  CUDA copies are asynchronous, so there is no thread: a write
(device -> host) is enqueued on `write_stream` behind the compute stream, a load
(host -> device) on `load_stream`; each returns a ticket whose event the cache polls
(`poll`) and which the compute stream waits on before a batch touches loaded pages
(`wait_loads`).
"""

from __future__ import annotations

import dataclasses
from typing import Any

import numpy as np
import torch

from .host_kv_pool import LRUHostKVPool


@dataclasses.dataclass
class Ticket:
    kind: str                      # "write" | "load"
    node_ids: list
    host_pages: np.ndarray
    device_pages: np.ndarray
    event: Any = None              # torch.cuda.Event or None (CPU: done at once)

    def done(self) -> bool:
        return self.event is None or self.event.query()


class HiCacheController:
    def __init__(self, host_pool: LRUHostKVPool, write_policy: str = "write_through"):
        self.host_pool = host_pool
        self.write_policy = write_policy
        self.on_gpu = host_pool.on_gpu
        self.write_stream = torch.cuda.Stream() if self.on_gpu else None
        self.load_stream = torch.cuda.Stream() if self.on_gpu else None
        self.pending: list[Ticket] = []
        self.unwaited_loads: list[Ticket] = []
        self.bytes_written = 0
        self.bytes_loaded = 0

    def _page_bytes(self) -> int:
        return sum(v.shape[1] * v.element_size() for v in self.host_pool.host_views)

    def write(self, node_id, device_pages: np.ndarray, host_pages: np.ndarray) -> Ticket:
        t = Ticket("write", [node_id], host_pages, device_pages)
        if self.on_gpu:
            self.write_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.write_stream):
                self.host_pool.backup_from_device(device_pages, host_pages)
                t.event = torch.cuda.Event()
                t.event.record()
        else:
            self.host_pool.backup_from_device(device_pages, host_pages)
        self.bytes_written += len(host_pages) * self._page_bytes()
        self.pending.append(t)
        return t

    def load(self, node_ids: list, host_pages: np.ndarray, device_pages: np.ndarray) -> Ticket:
        t = Ticket("load", list(node_ids), host_pages, device_pages)
        if self.on_gpu:
            # the target pages may still be read by work already queued on the compute stream
            self.load_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.load_stream):
                self.host_pool.load_to_device(host_pages, device_pages)
                t.event = torch.cuda.Event()
                t.event.record()
        else:
            self.host_pool.load_to_device(host_pages, device_pages)
        self.bytes_loaded += len(host_pages) * self._page_bytes()
        self.pending.append(t)
        self.unwaited_loads.append(t)
        return t

    def wait_loads(self) -> int:
        """Order the compute stream after every load issued so far; returns how many."""
        n = len(self.unwaited_loads)
        if self.on_gpu:
            cur = torch.cuda.current_stream()
            for t in self.unwaited_loads:
                cur.wait_event(t.event)
        self.unwaited_loads = []
        return n

    def poll(self) -> list[Ticket]:
        done = [t for t in self.pending if t.done()]
        if done:
            self.pending = [t for t in self.pending if not t.done()]
        return done

    def sync(self) -> None:
        """Block until every copy issued so far has finished (tickets stay pending until polled)."""
        if self.on_gpu:
            self.write_stream.synchronize()
            self.load_stream.synchronize()

    def drain(self) -> list[Ticket]:
        self.sync()
        return self.poll()
