"""Allocation helpers shared by the scheduler paths (reference `mem_cache/common.py`:
`alloc_token_slots` :13, `alloc_paged_token_slots_extend` :41, `evict_from_tree_cache` :72,
`available_and_evictable_str` :103, `release_kv_cache` :120)."""

from __future__ import annotations

import numpy as np


def evict_from_tree_cache(tree_cache, num_tokens: int, dp_rank: int = 0):
    """Ask the prefix cache to release `num_tokens` slots (both budgets for a sliding-window cache)."""
    if tree_cache is None or num_tokens <= 0:
        return 0
    if hasattr(tree_cache, "swa_evictable_size"):
        return tree_cache.evict(num_tokens, num_tokens)
    return tree_cache.evict(num_tokens, dp_rank=dp_rank)


def alloc_token_slots(tree_cache, allocator, num_tokens: int, dp_rank: int = 0) -> np.ndarray:
    """`num_tokens` slots (page aligned for paged allocators), evicting cached prefixes if needed."""
    if allocator.available_size(dp_rank) < num_tokens:
        evict_from_tree_cache(tree_cache, num_tokens - allocator.available_size(dp_rank), dp_rank)
    out = allocator.alloc(num_tokens, dp_rank=dp_rank)
    if out is None:
        raise RuntimeError(f"out of KV slots: need {num_tokens}. {available_and_evictable_str(tree_cache, allocator, dp_rank)}")
    return out


def alloc_paged_token_slots_extend(tree_cache, allocator, prefix_lens, seq_lens, last_loc, extend_num_tokens: int,
                                   dp_rank: int = 0) -> np.ndarray:
    page = allocator.page_size
    worst = extend_num_tokens + len(seq_lens) * page             # every request may open one extra page
    if allocator.available_size(dp_rank) < worst:
        evict_from_tree_cache(tree_cache, worst - allocator.available_size(dp_rank), dp_rank)
    out = allocator.alloc_extend(prefix_lens, seq_lens, last_loc, extend_num_tokens, dp_rank=dp_rank)
    if out is None:
        raise RuntimeError(f"out of KV slots: need {extend_num_tokens}. "
                           f"{available_and_evictable_str(tree_cache, allocator, dp_rank)}")
    return out


def available_and_evictable_str(tree_cache, allocator, dp_rank: int = 0) -> str:
    avail = allocator.available_size(dp_rank)
    if isinstance(avail, tuple):
        return f"available (full, swa) = {avail}"
    ev = tree_cache.evictable_size(dp_rank) if tree_cache is not None else 0
    return f"available = {avail}, evictable = {ev}, protected = {tree_cache.protected_size(dp_rank) if tree_cache else 0}"


def release_kv_cache(req, tree_cache, is_insert: bool = True):
    """Return a finished / aborted request's KV to the cache (shared part stays, the rest is freed)
    and its row to the request pool."""
    tree_cache.cache_finished_req(req, is_insert=is_insert)
    pool = tree_cache.req_to_token_pool
    if req.req_pool_idx is not None:
        pool.free(req.req_pool_idx)
        req.req_pool_idx = None
