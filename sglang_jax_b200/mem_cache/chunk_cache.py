"""Prefix "cache" that shares nothing: used with `--disable-radix-cache`
(reference `mem_cache/chunk_cache.py`).  It only keeps a chunked request's own
slots reachable between chunks and frees everything at finish."""

from __future__ import annotations

import numpy as np

from .base_prefix_cache import BasePrefixCache, MatchResult


class ChunkCache(BasePrefixCache):
    disable = True

    def __init__(self, req_to_token_pool, token_to_kv_pool_allocator, page_size: int = 1):
        self.req_to_token_pool = req_to_token_pool
        self.token_to_kv_pool_allocator = token_to_kv_pool_allocator
        self.page_size = page_size

    def reset(self):
        pass

    def match_prefix(self, key=None, **kw) -> MatchResult:
        return MatchResult(np.empty(0, np.int32), None, None)

    def cache_finished_req(self, req, **kw):
        kv = self.req_to_token_pool.read(req.req_pool_idx, req.committed_kv_len())
        self.token_to_kv_pool_allocator.free(kv.copy(), dp_rank=getattr(req, "dp_rank", 0) or 0)

    def cache_unfinished_req(self, req, **kw):
        req.prefix_indices = self.req_to_token_pool.read(req.req_pool_idx, len(req.fill_ids)).copy()
