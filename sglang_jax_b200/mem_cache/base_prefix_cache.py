"""Interface shared by the prefix caches (reference `mem_cache/base_prefix_cache.py`)."""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any

import numpy as np


@dataclass
class MatchResult:
    device_indices: np.ndarray      # KV slots of the matched prefix
    last_device_node: Any           # deepest node covering it (to lock)
    last_host_node: Any = None      # deepest node whose KV is on the host tier
    host_hit_length: int = 0


class BasePrefixCache(ABC):
    disable: bool = False

    @abstractmethod
    def reset(self): ...

    @abstractmethod
    def match_prefix(self, key, **kw) -> MatchResult: ...

    @abstractmethod
    def cache_finished_req(self, req, **kw): ...

    @abstractmethod
    def cache_unfinished_req(self, req, **kw): ...

    def insert(self, key, value=None, **kw): ...

    def evict(self, num_tokens: int, dp_rank: int = 0): ...

    def inc_lock_ref(self, node): return 0

    def dec_lock_ref(self, node): return 0

    def evictable_size(self, dp_rank: int = 0) -> int: return 0

    def protected_size(self, dp_rank: int = 0) -> int: return 0

    def total_size(self) -> int: return 0

    def pretty_print(self): ...

    def take_events(self): return []
