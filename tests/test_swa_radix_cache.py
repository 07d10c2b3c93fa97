"""Sliding-window radix cache: tombstones, window-aware matching, dual eviction and locks
(reference tests: `python/sgl_jax/test/mem_cache/test_swa_radix_cache.py`)."""

import numpy as np

from sglang_jax_b200.mem_cache.allocator import SWATokenToKVPoolAllocator
from sglang_jax_b200.mem_cache.memory_pool import ReqToTokenPool
from sglang_jax_b200.mem_cache.radix_cache import RadixKey
from sglang_jax_b200.mem_cache.swa_radix_cache import SWARadixCache


def _mk(window=4, full=64, swa=32, page=1):
    alloc = SWATokenToKVPoolAllocator(full, swa, page)
    r2t = ReqToTokenPool(8, 128, "cpu", page)
    return alloc, SWARadixCache(r2t, alloc, window, page)


def test_tombstone_limits_match_to_live_window():
    alloc, c = _mk(window=4)
    a = alloc.alloc(12)
    c.insert(RadixKey(list(range(12))), a)
    b = alloc.alloc(6)
    c.insert(RadixKey(list(range(8)) + [100, 101, 102, 103, 104, 105]), np.concatenate([a[:8], b]))
    # tree: [0..8) -> {[8..12), [100..106)}
    assert c.match_prefix(RadixKey(list(range(12)))).device_indices.tolist() == list(a)
    swa_before = alloc.swa_available_size()
    full_freed, swa_freed = c.evict(swa_num_tokens=8)
    assert swa_freed >= 8 and alloc.swa_available_size() >= swa_before + 8
    # the internal node [0..8) is the LRU internal candidate or the leaves went: whatever happened,
    # a match never ends right after a tombstone with fewer than `window` live tokens behind it
    res = c.match_prefix(RadixKey(list(range(12))))
    n = len(res.device_indices)
    assert n in (0, 12)
    if n == 12:
        # [8..12) is 4 live tokens = one full window behind the end: allowed
        assert res.device_indices.tolist() == list(a)


def test_internal_node_is_tombstoned_and_leaves_survive():
    alloc, c = _mk(window=3)
    a = alloc.alloc(10)
    c.insert(RadixKey(list(range(10))), a)
    b = alloc.alloc(5)
    c.insert(RadixKey(list(range(6)) + [50, 51, 52, 53, 54]), np.concatenate([a[:6], b]))
    # touch both leaves so that the shared internal node [0..6) is the least recently used
    c.match_prefix(RadixKey(list(range(10))))
    c.match_prefix(RadixKey(list(range(6)) + [50, 51, 52, 53, 54]))
    c.root_node.children[next(iter(c.root_node.children))].last_access_time = 0
    full_freed, swa_freed = c.evict(swa_num_tokens=6)
    assert (full_freed, swa_freed) == (0, 6)
    full, swa = c.total_size()
    assert full == 15 and swa == 9
    # both continuations still match in full: each leaf carries >= window live tokens
    assert len(c.match_prefix(RadixKey(list(range(10)))).device_indices) == 10
    assert len(c.match_prefix(RadixKey(list(range(6)) + [50, 51, 52, 53, 54])).device_indices) == 11
    # a query that ends inside the tombstone cannot use it
    assert len(c.match_prefix(RadixKey(list(range(6)) + [77])).device_indices) == 0
    # inserting the same prefix again with fresh slots revives the tombstone
    fresh = alloc.alloc(6)
    c.insert(RadixKey(list(range(6))), fresh, prev_prefix_len=0)
    assert c.total_size() == (15, 15)
    assert c.match_prefix(RadixKey(list(range(6)) + [77])).device_indices.tolist() == list(fresh)


def test_locks_protect_path_and_window():
    alloc, c = _mk(window=4)
    a = alloc.alloc(12)
    c.insert(RadixKey(list(range(12))), a)
    c.insert(RadixKey(list(range(6))), a[:6])          # split: [0..6) + [6..12)
    leaf = c.match_prefix(RadixKey(list(range(12)))).last_device_node
    uid = c.inc_lock_ref(leaf)
    assert c.full_protected_size() == 12 and c.full_evictable_size() == 0
    # only the window part (the 6-token leaf covers it) is SWA-locked
    assert c.swa_protected_size() == 6 and c.swa_evictable_size() == 6
    assert c.evict(full_num_tokens=12) == (0, 0)
    f, s = c.evict(swa_num_tokens=6)                    # the unlocked internal node becomes a tombstone
    assert (f, s) == (0, 6)
    c.dec_lock_ref(leaf, uid)
    assert c.full_protected_size() == 0 and c.swa_protected_size() == 0
    assert c.full_evictable_size() == 12 and c.swa_evictable_size() == 6
    f, s = c.evict(full_num_tokens=12)
    assert f == 12 and c.total_size() == (0, 0)
    assert alloc.full_available_size() == 64 and alloc.swa_available_size() == 32


def test_request_lifecycle_with_decode_time_swa_release():
    class Req:
        pass
    alloc, c = _mk(window=4, page=1)
    pool = c.req_to_token_pool
    r = Req()
    r.origin_input_ids, r.output_ids = list(range(10)), [90, 91, 92]
    r.extra_key, r.dp_rank, r.req_pool_idx = None, 0, 0
    r.last_matched_prefix_len, r.last_node, r.swa_evicted_seqlen = 0, c.root_node, 0
    slots = alloc.alloc(12)
    pool.write(0, 0, slots)
    r.committed_kv_len = lambda: 12
    # decoding at length 12 with window 4: tokens before 8 are out of every window
    assert c.evict_req_swa(r, 12) == 8
    assert alloc.swa_available_size() == 32 - 4
    c.cache_finished_req(r)
    assert c.total_size() == (12, 4)
    # the 4 live tokens at the end make the whole 12-token prefix matchable
    assert len(c.match_prefix(RadixKey(list(range(10)) + [90, 91])).device_indices) == 12
    assert len(c.match_prefix(RadixKey(list(range(10)))).device_indices) == 0
    c.evict(full_num_tokens=12)
    assert alloc.full_available_size() == 64 and alloc.swa_available_size() == 32
