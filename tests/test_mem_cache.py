"""Allocators, request table and radix cache (CPU)."""

import numpy as np
import pytest

from sglang_jax_b200.mem_cache.allocator import (PagedTokenToKVPoolAllocator, SWATokenToKVPoolAllocator,
                                                 TokenToKVPoolAllocator)
from sglang_jax_b200.mem_cache.memory_pool import ReqToTokenPool
from sglang_jax_b200.mem_cache.radix_cache import RadixCache, RadixKey


class FakeReq:
    def __init__(self, ids, pool_idx, extra_key=None, dp_rank=0):
        self.origin_input_ids = list(ids)
        self.output_ids = []
        self.fill_ids = list(ids)
        self.req_pool_idx = pool_idx
        self.prefix_indices = np.empty(0, np.int32)
        self.last_matched_prefix_len = 0
        self.last_node = None
        self.extra_key = extra_key
        self.dp_rank = dp_rank
        self.kv_len = len(ids)

    def committed_kv_len(self):
        return self.kv_len


def test_token_allocator_roundtrip():
    a = TokenToKVPoolAllocator(16)
    x = a.alloc(10)
    assert x.min() >= 1 and len(set(x.tolist())) == 10
    assert a.alloc(7) is None
    a.free(x[:4])
    assert a.available_size() == 10
    a.free_group_begin()
    a.free(x[4:6])
    assert a.available_size() == 10
    a.free_group_end()
    assert a.available_size() == 12


def test_paged_allocator_extend_and_decode():
    P = 4
    a = PagedTokenToKVPoolAllocator(64, P)
    # request with empty prefix, 6 tokens -> 2 pages, slots contiguous within pages
    out = a.alloc_extend([0], [6], [-1], 6)
    assert len(out) == 6 and out[0] % P == 0 and out[0] >= P
    assert (np.diff(out[:4]) == 1).all() and out[4] % P == 0
    # continue: prefix 6 (last page half full) + 5 tokens: first 2 go into the old page
    out2 = a.alloc_extend([6], [11], [int(out[-1])], 5)
    assert out2[0] == out[-1] + 1 and out2[1] == out[-1] + 2 and out2[2] % P == 0
    # decode: seq_len 12 -> token index 11 stays in the page; seq_len 13 opens a new page
    d = a.alloc_decode([12], [int(out2[-1])])
    assert d[0] == out2[-1] + 1
    d2 = a.alloc_decode([13], [int(d[0])])
    assert d2[0] % P == 0 and d2[0] != d[0] + 1 or d2[0] == d[0] + 1  # new page anywhere
    before = a.available_size()
    a.free(np.concatenate([out, out2, d, d2]))
    assert a.available_size() == before + 4 * P
    assert a.available_size() == 64


def test_paged_allocator_oom_is_atomic():
    a = PagedTokenToKVPoolAllocator(8, 4)
    assert a.alloc_extend([0, 0], [5, 5], [-1, -1], 10) is None
    assert a.available_size() == 8


def test_swa_allocator_pairs_and_early_free():
    a = SWATokenToKVPoolAllocator(32, 16, 4)
    x = a.alloc(8)
    assert (a.translate_loc_from_full_to_swa(x) > 0).all()
    swa_before = a.swa_available_size()
    a.free_swa(x[:4])
    assert a.swa_available_size() == swa_before + 4
    a.free(x)
    assert a.full_available_size() == 32 and a.swa_available_size() == 16


def test_req_to_token_pool_page_deltas():
    pool = ReqToTokenPool(4, 64, "cpu", page_size=4)
    r = pool.alloc(1)[0]
    pool.write(r, 0, np.arange(8, 14))
    rows, pos, ids = pool.take_page_deltas()
    assert rows.tolist() == [r, r] and pos.tolist() == [0, 1] and ids.tolist() == [2, 3]
    pool.set_one(r, 6, 14)
    assert pool.take_page_deltas()[0].size == 0       # same page, no delta
    pool.set_one(r, 8, 40)
    rows, pos, ids = pool.take_page_deltas()
    assert pos.tolist() == [2] and ids.tolist() == [10]


def _mk(page=1, size=256):
    pool = ReqToTokenPool(16, 128, "cpu", page)
    alloc = TokenToKVPoolAllocator(size) if page == 1 else PagedTokenToKVPoolAllocator(size, page)
    return pool, alloc, RadixCache(pool, alloc, page)


def test_radix_insert_match_split():
    _, _, c = _mk()
    assert c.insert(RadixKey([1, 2, 3, 4]), np.array([10, 11, 12, 13])) == 0
    assert c.insert(RadixKey([1, 2, 5, 6]), np.array([10, 11, 20, 21])) == 2
    m = c.match_prefix(RadixKey([1, 2, 3, 9]))
    assert m.device_indices.tolist() == [10, 11, 12]
    assert c.total_size() == 6
    assert c.match_prefix(RadixKey([7])).device_indices.size == 0


def test_radix_paged_alignment():
    _, _, c = _mk(page=4)
    ids = list(range(10))
    c.insert(RadixKey(ids), np.arange(100, 110))
    assert c.total_size() == 8                      # only whole pages are stored
    assert len(c.match_prefix(RadixKey(ids[:7])).device_indices) == 4
    assert len(c.match_prefix(RadixKey([0, 1, 2, 9, 9, 9, 9, 9])).device_indices) == 0


def test_radix_namespaces():
    _, _, c = _mk()
    c.insert(RadixKey([1, 2, 3], extra_key="a"), np.array([1, 2, 3]))
    c.insert(RadixKey([1, 2, 3], dp_rank=1), np.array([4, 5, 6]))
    assert c.match_prefix(RadixKey([1, 2, 3])).device_indices.size == 0
    assert c.match_prefix(RadixKey([1, 2, 3], extra_key="a")).device_indices.tolist() == [1, 2, 3]
    assert c.match_prefix(RadixKey([1, 2, 3], dp_rank=1)).device_indices.tolist() == [4, 5, 6]
    assert c.evictable_size(1) == 3 and c.evictable_size(0) == 3 and c.evictable_size() == 6


def test_radix_lock_and_evict_lru():
    _, alloc, c = _mk()
    a = alloc.alloc(4)
    b = alloc.alloc(4)
    c.insert(RadixKey([1, 2, 3, 4]), a)
    c.insert(RadixKey([5, 6, 7, 8]), b)
    node_a = c.match_prefix(RadixKey([1, 2, 3, 4])).last_device_node
    c.inc_lock_ref(node_a)
    assert c.protected_size() == 4 and c.evictable_size() == 4
    free0 = alloc.available_size()
    c.evict(100)
    assert alloc.available_size() == free0 + 4      # only the unlocked branch went away
    assert c.match_prefix(RadixKey([1, 2, 3, 4])).device_indices.tolist() == a.tolist()
    c.dec_lock_ref(node_a)
    c.evict(100)
    assert alloc.available_size() == 256 and c.total_size() == 0


def test_radix_request_lifecycle_frees_duplicates():
    pool, alloc, c = _mk(page=4, size=64)
    ids = list(range(1, 11))                        # 10 tokens: 2 whole pages + tail of 2
    reqs = []
    for i in range(2):
        r = FakeReq(ids, pool.alloc(1)[0])
        slots = alloc.alloc_extend([0], [10], [-1], 10)
        pool.write(r.req_pool_idx, 0, slots)
        r.last_node = c.root_node
        reqs.append((r, slots))
    c.cache_finished_req(reqs[0][0])
    pool.free(reqs[0][0].req_pool_idx)
    assert c.total_size() == 8
    c.cache_finished_req(reqs[1][0])                # duplicate pages + both tails are returned
    pool.free(reqs[1][0].req_pool_idx)
    assert alloc.available_size() + c.evictable_size() == 64
    assert c.protected_size() == 0


def test_radix_unfinished_req_rewrites_to_canonical_slots():
    pool, alloc, c = _mk(page=4, size=64)
    ids = list(range(1, 10))
    r1 = FakeReq(ids, pool.alloc(1)[0])
    s1 = alloc.alloc_extend([0], [9], [-1], 9)
    pool.write(r1.req_pool_idx, 0, s1)
    r1.last_node = c.root_node
    c.cache_unfinished_req(r1)
    assert r1.last_matched_prefix_len == 8 and len(r1.prefix_indices) == 9
    r2 = FakeReq(ids, pool.alloc(1)[0])
    s2 = alloc.alloc_extend([0], [9], [-1], 9)
    pool.write(r2.req_pool_idx, 0, s2)
    r2.last_node = c.root_node
    c.cache_unfinished_req(r2)
    # r2 now points at r1's pages for the shared part; its own duplicate pages are free again
    assert pool.read(r2.req_pool_idx, 8).tolist() == s1[:8].tolist()
    assert pool.read(r2.req_pool_idx, 9)[8] == s2[8]
    assert c.protected_size() == 8
    for r in (r1, r2):
        c.cache_finished_req(r)
        pool.free(r.req_pool_idx)
    assert alloc.available_size() + c.evictable_size() == 64 and c.protected_size() == 0
