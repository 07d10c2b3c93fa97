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


def _unified(policy="write_through", host_pages=16, size=64, page=4, snaps=4):
    from sglang_jax_b200.mem_cache.unified_radix_cache import UnifiedHiRadixCache
    pool = MHATokenToKVPool(size, page, torch.float32, 2, 8, 2, "cpu")
    alloc = PagedTokenToKVPoolAllocator(size, page, kvcache=pool)
    r2t = ReqToTokenPool(8, 128, "cpu", page)
    cache = UnifiedHiRadixCache(r2t, alloc, page, pool, num_request_slots=8, num_snapshot_slots=snaps,
                                write_policy=policy, host_pages=host_pages)
    return pool, alloc, cache


def _checkpoint(cache, tokens):
    """Attach a snapshot slot to the node that ends exactly at `tokens` (what a tracked prefill step does)."""
    values, node = cache._match(tokens, RadixKey(tokens).namespace)
    assert sum(len(v) for v in values) == len(tokens)
    slot = cache._alloc_snapshot()
    cache._snap[node.id], cache._nodes[node.id], cache._lru[node.id] = slot, node, None
    return node, slot


def test_unified_tree_with_host_tier_matches_through_host_only_nodes_to_a_checkpoint():
    """Hybrid (recurrent + full attention) prefix cache over the host tier: the KV of a checkpointed prefix is demoted
    to the host, the checkpoint stays; a later match reports the host hit, the load-back returns the KV bit-exact and
    the request ends on the checkpoint node.  Reference: the HiCache hooks of `unified_radix_cache.py`."""
    from types import SimpleNamespace
    pool, alloc, cache = _unified()
    toks = list(range(100, 116))
    slots = alloc.alloc(16)
    data = _fill(pool, slots, 5)
    cache.insert(RadixKey(toks[:8]), slots[:8])
    cache.insert(RadixKey(toks), slots)
    cache.check_hicache_events()
    n8, s8 = _checkpoint(cache, toks[:8])
    n16, s16 = _checkpoint(cache, toks)
    # a match ends on the deepest checkpoint (here the whole key), not past it
    req = SimpleNamespace(recurrent_cow_src=None)
    res = cache.match_prefix(RadixKey(toks + [1, 2, 3, 4]), req=req)
    assert len(res.device_indices) == 16 and res.last_device_node is n16 and req.recurrent_cow_src == s16
    # evict the lower half of the chain from the device: it stays in the tree as a host-only node with its checkpoint
    assert cache.evict(8) == 8 and n16.evicted and n16.backuped and n16.id in cache._snap
    for b in pool.kv_buffer:
        b.zero_()
    pool_data = _fill(pool, slots[:8], 6)          # the upper half is still on the device
    req = SimpleNamespace(recurrent_cow_src=None)
    res = cache.match_prefix(RadixKey(toks + [1, 2, 3, 4]), req=req)
    assert res.device_indices.tolist() == list(slots[:8]) and res.last_device_node is n8
    assert res.last_host_node is n16 and res.host_hit_length == 8 and req.recurrent_cow_src == s8
    new_slots, last = cache.init_load_back(res.last_host_node, res.host_hit_length)
    cache.ready_to_load_host_cache()
    cache.check_hicache_events()
    assert last is n16 and len(new_slots) == 8
    _check(pool, new_slots, [(k[8:], v[8:]) for k, v in data])
    # the scheduler now points the request at the deeper node: its checkpoint is the one that gets cloned
    req2 = SimpleNamespace(recurrent_cow_src=s8, prefix_indices=np.arange(16), last_node=last, req_pool_idx=3)
    cache.on_request_scheduled(req2)
    assert cache.take_recurrent_copies() == [(s16, 4)]
    cache.assert_recurrent_slot_ledger()
    del pool_data


def test_unified_host_tier_spans_device_nodes_between_checkpoint_and_host_chain_and_frees_snapshots():
    from types import SimpleNamespace
    pool, alloc, cache = _unified(host_pages=8)
    toks = list(range(200, 224))
    slots = alloc.alloc(24)
    data = _fill(pool, slots, 7)
    for n in (8, 16, 24):
        cache.insert(RadixKey(toks[:n]), slots[:n])
    cache.check_hicache_events()
    n8, s8 = _checkpoint(cache, toks[:8])
    n24, s24 = _checkpoint(cache, toks)             # no checkpoint on the middle node [8, 16)
    assert cache.evict(8) == 8 and n24.evicted
    req = SimpleNamespace(recurrent_cow_src=None)
    res = cache.match_prefix(RadixKey(toks + [9, 9, 9, 9]), req=req)
    # device part up to the device checkpoint (8 tokens); the host hit spans the middle device node and the host node
    assert len(res.device_indices) == 8 and res.last_device_node is n8 and res.last_host_node is n24
    assert res.host_hit_length == 16
    new_slots, last = cache.init_load_back(res.last_host_node, res.host_hit_length)
    cache.ready_to_load_host_cache()
    cache.check_hicache_events()
    assert last is n24 and len(new_slots) == 16 and new_slots[:8].tolist() == list(slots[8:16])
    _check(pool, new_slots[8:], [(k[16:], v[16:]) for k, v in data])
    # without a checkpoint anywhere on the path nothing can be reused
    other = list(range(300, 308))
    o = alloc.alloc(8)
    cache.insert(RadixKey(other), o)
    assert len(cache.match_prefix(RadixKey(other + [1] * 4)).device_indices) == 0
    # host eviction of a checkpointed host-only node returns its snapshot slot
    cache.check_hicache_events()
    cache.evict(64)
    before = cache.snapshot_slots_in_use()
    assert before == 2
    cache.evict_host(64)
    assert cache.snapshot_slots_in_use() == 0 and cache.host_size_pages() == 0
    cache.assert_recurrent_slot_ledger()


def test_engine_hybrid_model_restarts_from_a_checkpoint_whose_kv_came_back_from_the_host(tmp_path):
    """A Qwen3-Next-style hybrid under memory pressure: the first prompt's KV is demoted to the host tier while its
    recurrent-state checkpoint stays on the device; repeating the prompt loads the KV back, clones the checkpoint and
    produces exactly the tokens of a run without any cache."""
    import json
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.parallel import state as ps
    cfg = dict(architectures=["Qwen3NextForCausalLM"], model_type="qwen3_next", hidden_size=64, intermediate_size=96,
               num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6,
               vocab_size=256, max_position_embeddings=512, full_attention_interval=2, linear_num_key_heads=2,
               linear_num_value_heads=4, linear_key_head_dim=8, linear_value_head_dim=8, linear_conv_kernel_dim=4,
               partial_rotary_factor=0.5, num_experts=0, tie_word_embeddings=False, torch_dtype="float32",
               layer_types=["linear_attention", "full_attention"] * 2)
    path = tmp_path / "q3n"
    path.mkdir()
    (path / "config.json").write_text(json.dumps(cfg))
    rng = np.random.RandomState(1)
    prompts = [rng.randint(5, 250, size=97).tolist() for _ in range(4)]
    sp = {"temperature": 0.0, "max_new_tokens": 6, "ignore_eos": True}

    def run(**kw):
        ps.reset_state()
        eng = Engine(model_path=str(path), device="cpu", enable_single_process=True, page_size=16,
                     skip_tokenizer_init=True, max_total_tokens=256, dtype="float32", log_level="error",
                     max_running_requests=1, load_format="dummy", **kw)
        try:
            outs = [eng.generate(input_ids=p, sampling_params=sp) for p in prompts + prompts[:1]]
            tc = eng.scheduler.tree_cache
            if hasattr(tc, "assert_recurrent_slot_ledger"):
                tc.assert_recurrent_slot_ledger()
            eng.scheduler.check_memory()
            return outs, tc
        finally:
            eng.shutdown()

    base, _ = run(disable_radix_cache=True)
    hi, tc = run(hicache_storage="host", hicache_ratio=4.0, recurrent_snapshot_slots=8)
    assert type(tc).__name__ == "UnifiedHiRadixCache"
    assert [o["output_ids"] for o in hi] == [o["output_ids"] for o in base]
    # the checkpoint at the last page boundary of the first prompt (96 tokens) was reused through the host tier
    assert hi[-1]["meta_info"]["cached_tokens"] == 96
    assert tc.controller.bytes_loaded > 0
