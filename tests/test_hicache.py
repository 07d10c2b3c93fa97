"""Host-memory KV tier on CPU: pages survive device eviction and come back bit-exact
(reference tests: `python/sgl_jax/test/mem_cache/test_host_kv_pool.py`, HiCache e2e)."""

import numpy as np
import pytest
import torch

from sglang_jax_b200.mem_cache.allocator import PagedTokenToKVPoolAllocator
from sglang_jax_b200.mem_cache.hiradix_cache import HiRadixCache
from sglang_jax_b200.mem_cache.host_kv_pool import QueueHostKVPool
from sglang_jax_b200.mem_cache.memory_pool import MHATokenToKVPool, ReqToTokenPool
from sglang_jax_b200.mem_cache.radix_cache import RadixKey


def _setup(policy="write_through", threshold=1, host_pages=16, size=64, page=4):
    pool = MHATokenToKVPool(size, page, torch.float32, 2, 8, 2, "cpu")
    alloc = PagedTokenToKVPoolAllocator(size, page, kvcache=pool)
    r2t = ReqToTokenPool(8, 128, "cpu", page)
    cache = HiRadixCache(r2t, alloc, page, pool, write_policy=policy, write_through_threshold=threshold,
                         host_pages=host_pages)
    return pool, alloc, cache


def _fill(pool, slots, seed):
    g = torch.Generator().manual_seed(seed)
    loc = torch.as_tensor(slots, dtype=torch.long)
    data = []
    for layer in range(pool.layer_num):
        k = torch.randn(len(slots), pool.head_num, pool.head_dim, generator=g)
        v = torch.randn(len(slots), pool.head_num, pool.head_dim, generator=g)
        pool.set_kv_buffer(layer, loc, k, v)
        data.append((k, v))
    return data


def _check(pool, slots, data):
    loc = torch.as_tensor(slots, dtype=torch.long)
    for layer, (k, v) in enumerate(data):
        gk, gv = pool.gather(layer, loc)
        assert torch.equal(gk, k) and torch.equal(gv, v)


def test_backup_evict_load_back_roundtrip():
    pool, alloc, cache = _setup()
    toks = list(range(100, 116))
    slots = alloc.alloc(16)
    data = _fill(pool, slots, 1)
    cache.insert(RadixKey(toks), slots)
    cache.check_hicache_events()
    assert cache.host_size_pages() == 4
    assert cache.evict(16) == 16 and alloc.available_size() == 64
    for b in pool.kv_buffer:
        b.zero_()
    res = cache.match_prefix(RadixKey(toks + [1, 2, 3, 4]))
    assert len(res.device_indices) == 0 and res.host_hit_length == 16
    new_slots, node = cache.init_load_back(res.last_host_node, res.host_hit_length)
    assert len(new_slots) == 16
    cache.ready_to_load_host_cache()
    cache.check_hicache_events()
    _check(pool, new_slots, data)
    res2 = cache.match_prefix(RadixKey(toks))
    assert res2.device_indices.tolist() == list(new_slots) and res2.host_hit_length == 0
    assert node.lock_ref == 0 and cache.evictable_size() == 16


def test_partial_host_hit_splits_host_pages():
    pool, alloc, cache = _setup()
    toks = list(range(16))
    slots = alloc.alloc(16)
    data = _fill(pool, slots, 2)
    cache.insert(RadixKey(toks), slots)
    cache.check_hicache_events()
    cache.evict(16)
    # only the first 8 tokens match
    res = cache.match_prefix(RadixKey(toks[:8] + [99] * 8))
    assert res.host_hit_length == 8
    new_slots, _ = cache.init_load_back(res.last_host_node, 8)
    cache.check_hicache_events()
    _check(pool, new_slots, [(k[:8], v[:8]) for k, v in data])
    # the tail is still only on the host and still loadable
    res = cache.match_prefix(RadixKey(toks))
    assert len(res.device_indices) == 8 and res.host_hit_length == 8
    tail_slots, _ = cache.init_load_back(res.last_host_node, 8)
    cache.check_hicache_events()
    _check(pool, tail_slots, [(k[8:], v[8:]) for k, v in data])


def test_selective_write_through_and_write_back_and_host_eviction():
    pool, alloc, cache = _setup(policy="write_through_selective", threshold=2)
    toks = list(range(8))
    slots = alloc.alloc(8)
    cache.insert(RadixKey(toks), slots)
    cache.check_hicache_events()
    assert cache.host_size_pages() == 0           # one hit: not hot enough yet
    cache.insert(RadixKey(toks), slots)
    cache.check_hicache_events()
    assert cache.host_size_pages() == 2
    # write_back: nothing is copied until the device evicts
    pool, alloc, cache = _setup(policy="write_back", host_pages=4)
    a, b = alloc.alloc(8), alloc.alloc(16)
    da = _fill(pool, a, 3)
    cache.insert(RadixKey(list(range(8))), a)
    cache.insert(RadixKey(list(range(50, 66))), b)
    assert cache.host_size_pages() == 0
    cache.evict(8)                                # LRU: the first key goes to the host
    assert cache.host_size_pages() == 2
    res = cache.match_prefix(RadixKey(list(range(8))))
    assert res.host_hit_length == 8
    # the host tier is full after the second eviction: its LRU entry is dropped for good
    cache.evict(16)
    assert cache.host_size_pages() == 4
    assert cache.match_prefix(RadixKey(list(range(8)))).host_hit_length == 0
    del da


def test_queue_pool_fifo_staging():
    pool = MHATokenToKVPool(32, 4, torch.float32, 1, 4, 1, "cpu")
    q = QueueHostKVPool(pool, 4)
    slots = np.arange(4, 12)
    data = _fill(pool, slots, 5)
    assert q.put("req-1", np.array([1, 2]))
    assert not q.put("req-2", np.array([1, 2, 3]))       # only two pages left
    pool.kv_buffer[0].zero_()
    assert q.get("req-1", np.array([5, 6]))
    _check(pool, np.arange(20, 28), data)
    assert q.available_pages() == 4 and not q.get("req-1", np.array([5, 6]))


def test_engine_reuses_prefix_from_host_tier(tmp_path):
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import write_tiny_qwen3_checkpoint
    ckpt = write_tiny_qwen3_checkpoint(str(tmp_path / "m"))
    rng = np.random.RandomState(0)
    prompts = [rng.randint(5, 1000, size=96).tolist() for _ in range(4)]
    sp = {"temperature": 0.0, "max_new_tokens": 6, "ignore_eos": True}

    def run(**kw):
        ps.reset_state()
        eng = Engine(model_path=ckpt, device="cpu", enable_single_process=True, page_size=16, skip_tokenizer_init=True,
                     max_total_tokens=256, dtype="float32", log_level="error", max_running_requests=1, **kw)
        try:
            outs = []
            for p in prompts + prompts[:1]:
                outs.append(eng.generate(input_ids=p, sampling_params=sp))
            return outs, eng.scheduler
        finally:
            eng.shutdown()

    base, _ = run()
    hi, sched = run(hicache_storage="host", hicache_ratio=4.0)
    assert [o["output_ids"] for o in hi] == [o["output_ids"] for o in base]
    # 256 device tokens cannot hold four 96-token prompts: the first one was evicted and came back from the host
    assert base[-1]["meta_info"]["cached_tokens"] == 0
    assert hi[-1]["meta_info"]["cached_tokens"] >= 80
    assert sched.tree_cache.controller.bytes_loaded > 0
