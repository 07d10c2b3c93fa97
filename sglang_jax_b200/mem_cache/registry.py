"""Chooses the slot allocator and the prefix cache for a model / server configuration (reference
`mem_cache/registry.py`: `TreeCacheBuildContext` :18, `create_tree_cache` :122).

Factories are looked up by name so a deployment can register its own (`register_tree_cache`);
`default_radix_cache_factory` implements the built-in rules:

* sliding-window hybrid KV pool      -> `SWARadixCache` over the dual allocator
* `--disable-radix-cache`            -> `ChunkCache`
* recurrent (linear-attention) model -> `UnifiedRadixCache` (needs snapshot slots, else no sharing);
  with `--hicache-storage` `UnifiedHiRadixCache`
* `--hicache-storage`                -> `HiRadixCache`
* otherwise                          -> radix tree (C++ when built)
"""

from __future__ import annotations

import dataclasses
import logging
from typing import Any, Callable

from .base_prefix_cache import BasePrefixCache
from .cache_init_params import CacheInitParams

logger = logging.getLogger(__name__)


@dataclasses.dataclass
class TreeCacheBuildContext:
    server_args: Any
    model_config: Any
    req_to_token_pool: Any
    kv_pool: Any
    max_total_num_tokens: int
    page_size: int
    spec_algorithm: str | None = None
    recurrent_pool: Any = None


@dataclasses.dataclass
class TreeCacheBuildResult:
    allocator: Any
    tree_cache: BasePrefixCache
    needs_sequential_schedule: bool = False      # the cache cannot tolerate the overlap loop's extra step


_FACTORIES: dict[str, Callable[[TreeCacheBuildContext], TreeCacheBuildResult]] = {}


def register_tree_cache(name: str, factory: Callable[[TreeCacheBuildContext], TreeCacheBuildResult]):
    _FACTORIES[name] = factory


def is_recurrent(ctx: TreeCacheBuildContext) -> bool:
    lt = getattr(getattr(ctx.model_config, "hf_text_config", None), "layer_types", None) or []
    return ctx.recurrent_pool is not None or "linear_attention" in lt


def default_radix_cache_factory(ctx: TreeCacheBuildContext) -> TreeCacheBuildResult:
    from . import native as native_sched
    from .chunk_cache import ChunkCache
    sa, kv, rp = ctx.server_args, ctx.kv_pool, ctx.recurrent_pool
    recurrent = is_recurrent(ctx)
    if recurrent and not sa.disable_radix_cache and (rp is None or rp.snapshot_slots <= 0):
        # a shared prefix needs the recurrent state at its end: checkpoints live in the snapshot area
        logger.info("hybrid linear-attention model: prefix sharing is off (needs --recurrent-snapshot-slots > 0)")
        sa.disable_radix_cache = True
    if kv is not None and hasattr(kv, "swa_pool"):
        from .allocator import SWATokenToKVPoolAllocator
        from .swa_radix_cache import SWARadixCache
        alloc = SWATokenToKVPoolAllocator(kv.size, kv.size_swa, ctx.page_size, kvcache=kv)
        return TreeCacheBuildResult(alloc, SWARadixCache(ctx.req_to_token_pool, alloc,
                                                         ctx.model_config.sliding_window or 4096, ctx.page_size,
                                                         disable=sa.disable_radix_cache))
    alloc = native_sched.make_allocator(ctx.max_total_num_tokens, ctx.page_size, kv)
    p = CacheInitParams(ctx.req_to_token_pool, alloc, ctx.page_size, enable_kv_cache_events=bool(sa.kv_events_config),
                        is_eagle=ctx.spec_algorithm in ("EAGLE", "EAGLE3"), kv_pool=kv)
    if sa.disable_radix_cache:
        return TreeCacheBuildResult(alloc, ChunkCache(p.req_to_token_pool, alloc, p.page_size))
    if recurrent or getattr(sa, "enable_unified_radix_tree", False):
        # `--enable-unified-radix-tree` (reference `mem_cache/registry.py`): the unified tree for every model; without
        # linear-attention layers it carries the FULL component only
        from .unified_radix_cache import UnifiedHiRadixCache, UnifiedRadixCache
        snap = dict(num_request_slots=rp.size if rp is not None else 0,
                    num_snapshot_slots=rp.snapshot_slots if rp is not None else 0,
                    enable_kv_cache_events=p.enable_kv_cache_events,
                    track_interval=getattr(sa, "recurrent_track_interval", None),
                    commit_on_finish=bool(sa.disable_overlap_schedule), recurrent=recurrent)
        if sa.hicache_storage != "disable" and kv is not None:
            # KV of the full-attention layers gets the host tier; checkpoints of the recurrent state stay on the device
            cache = UnifiedHiRadixCache(p.req_to_token_pool, alloc, p.page_size, kv, hicache_ratio=sa.hicache_ratio,
                                        write_policy=sa.hicache_write_policy,
                                        write_through_threshold=sa.hicache_write_through_threshold, **snap)
        else:
            cache = UnifiedRadixCache(p.req_to_token_pool, alloc, p.page_size, **snap)
        # checkpoints taken inside prefill steps are safe under overlap scheduling; the one at the end of a finished
        # request reads the request's own slot, which an overlapped extra decode step may already have advanced, so
        # it is only taken when the schedule is sequential
        return TreeCacheBuildResult(alloc, cache)
    if sa.hicache_storage != "disable" and kv is not None:
        from .hiradix_cache import HiRadixCache
        return TreeCacheBuildResult(alloc, HiRadixCache(p.req_to_token_pool, alloc, p.page_size, kv, sa.hicache_ratio,
                                                        sa.hicache_write_policy, sa.hicache_write_through_threshold))
    return TreeCacheBuildResult(alloc, native_sched.make_radix_cache(
        p.req_to_token_pool, alloc, p.page_size, enable_kv_cache_events=p.enable_kv_cache_events, is_eagle=p.is_eagle))


register_tree_cache("default", default_radix_cache_factory)


def create_tree_cache(ctx: TreeCacheBuildContext, name: str = "default") -> TreeCacheBuildResult:
    if name not in _FACTORIES:
        raise ValueError(f"unknown prefix-cache factory {name!r}; registered: {sorted(_FACTORIES)}")
    return _FACTORIES[name](ctx)
