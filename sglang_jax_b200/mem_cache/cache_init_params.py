"""What a prefix cache needs to be built (reference `mem_cache/cache_init_params.py`)."""

from __future__ import annotations

import dataclasses
from typing import Any


@dataclasses.dataclass
class CacheInitParams:
    req_to_token_pool: Any
    token_to_kv_pool_allocator: Any
    page_size: int
    disable: bool = False
    is_eagle: bool = False
    enable_kv_cache_events: bool = False
    sliding_window_size: int | None = None
    # hybrid recurrent models: request slots / checkpoint slots of the recurrent state pool
    num_recurrent_request_slots: int = 0
    num_recurrent_snapshot_slots: int = 0
    # hierarchical cache
    kv_pool: Any = None
    hicache_ratio: float = 2.0
    hicache_write_policy: str = "write_through"
    hicache_write_through_threshold: int = 1
