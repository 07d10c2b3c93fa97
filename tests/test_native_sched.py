"""The C++ paged allocator and radix tree behave exactly like the Python ones (randomised
operation sequences), and the serving engine produces the same tokens with either."""

import itertools
import random

import numpy as np
import pytest

from sglang_jax_b200.csrc.sched import build as sched_build

sched_build.build()

from sglang_jax_b200.mem_cache import native, radix_cache as rc  # noqa: E402
from sglang_jax_b200.mem_cache.allocator import PagedTokenToKVPoolAllocator, TokenToKVPoolAllocator  # noqa: E402
from sglang_jax_b200.mem_cache.radix_cache import RadixCache, RadixKey  # noqa: E402


class _Alloc:
    def __init__(self):
        self.freed = []

    def free(self, v, dp_rank=0):
        self.freed.append((dp_rank, np.sort(np.asarray(v)).tolist()))


@pytest.mark.parametrize("page", [1, 4])
def test_radix_tree_matches_python_tree(page, monkeypatch):
    assert native.available()
    tick = itertools.count()
    monkeypatch.setattr(rc.time, "monotonic", lambda: next(tick))      # strict LRU order on both sides
    rng = random.Random(page)
    fa, fb = _Alloc(), _Alloc()
    a, b = RadixCache(None, fa, page, enable_kv_cache_events=True), native.NativeRadixCache(None, fb, page, enable_kv_cache_events=True)
    locks, slot = [], 1
    for it in range(4000):
        op = rng.random()
        base = [rng.randrange(4) for _ in range(rng.randrange(1, 40))]
        key = RadixKey(base, rng.choice([None, "x"]), rng.choice([0, 1]))
        if op < 0.45:
            vals = np.arange(slot, slot + len(base), dtype=np.int32)
            slot += len(base)
            assert a.insert(key, vals) == b.insert(key, vals), it
        elif op < 0.8:
            ra, rb = a.match_prefix(key), b.match_prefix(key)
            assert ra.device_indices.tolist() == rb.device_indices.tolist(), it
            assert len(ra.device_indices) % page == 0
            if rng.random() < 0.3:
                assert a.inc_lock_ref(ra.last_device_node) == b.inc_lock_ref(rb.last_device_node)
                locks.append((ra.last_device_node, rb.last_device_node))
        elif op < 0.9 and locks:
            la, lb = locks.pop(rng.randrange(len(locks)))
            assert a.dec_lock_ref(la) == b.dec_lock_ref(lb)
        else:
            fa.freed.clear()
            fb.freed.clear()
            k, dp = rng.randrange(1, 60), rng.choice([None, 0, 1])
            assert a.evict(k, dp) == b.evict(k, dp), it
            assert fa.freed == fb.freed, it                                # same leaves, same order
        for dp in (None, 0, 1):
            assert a.evictable_size(dp) == b.evictable_size(dp), (it, dp)
            assert a.protected_size(dp) == b.protected_size(dp)
        assert a.total_size() == b.total_size()
    assert sorted(a.all_values_flatten().tolist()) == sorted(b.all_values_flatten().tolist())
    ea, eb = a.take_events(), b.take_events()
    assert [e["type"] for e in ea] == [e["type"] for e in eb] and len(ea) > 100
    assert [e.get("num_tokens") for e in ea] == [e.get("num_tokens") for e in eb]
    # handles: children / parent walk (what the DFS-weight policy uses)
    root = b.root_node
    kids = list(root.children.values())
    assert kids and all(k.parent == root for k in kids) and root.parent is None
    free_leaf = next((k for k in kids if k.lock_ref == 0), None)
    if free_leaf is not None:
        with pytest.raises(RuntimeError):
            b.dec_lock_ref(free_leaf)                                      # unlocking below zero is refused


@pytest.mark.parametrize("page", [1, 4, 16])
def test_allocator_matches_python_allocator(page):
    rng = random.Random(page)
    pa = TokenToKVPoolAllocator(2048) if page == 1 else PagedTokenToKVPoolAllocator(2048, page)
    na = native.NativePagedAllocator(2048, page)
    held = []

    def same(x, y):
        assert (x is None) == (y is None)
        if x is not None:
            assert np.asarray(x).tolist() == np.asarray(y).tolist()
        return x

    for it in range(3000):
        op = rng.random()
        if op < 0.25:
            n = rng.randrange(0, 5) * page
            x = same(pa.alloc(n), na.alloc(n))
            if x is not None and len(x):
                held.append(np.asarray(x))
        elif op < 0.55:
            B = rng.randrange(1, 5)
            pre = np.array([rng.randrange(0, 20) for _ in range(B)])
            ext = np.array([rng.randrange(0, 20) for _ in range(B)])
            last = np.where(pre > 0, rng.randrange(1, 100) * page + (pre - 1) % page, -1)
            x = same(pa.alloc_extend(pre, pre + ext, last, int(ext.sum())),
                     na.alloc_extend(pre, pre + ext, last, int(ext.sum())))
            if x is not None and len(x):
                held.append(np.asarray(x)[np.asarray(x) // page != (last.max() // page if page > 1 else -5)])
        elif op < 0.7:
            B = rng.randrange(1, 6)
            seq = np.array([rng.randrange(1, 50) for _ in range(B)])
            last = np.array([rng.randrange(1, 100) * page + (s - 2) % page for s in seq])
            same(pa.alloc_decode(seq, last), na.alloc_decode(seq, last))
        elif op < 0.75:
            pa.free_group_begin()
            na.free_group_begin()
            for _ in range(min(2, len(held))):
                h = held.pop(rng.randrange(len(held)))
                pa.free(h)
                na.free(h)
            assert pa.available_size() == na.available_size()
            pa.free_group_end()
            na.free_group_end()
        elif held:
            h = held.pop(rng.randrange(len(held)))
            pa.free(h)
            na.free(h)
        assert pa.available_size() == na.available_size(), it
        assert np.asarray(pa.backup_state()).tolist() == np.asarray(na.backup_state()).tolist(), it
    st = na.backup_state()
    na.alloc(page * 3)
    na.restore_state(st)
    assert na.backup_state().tolist() == st.tolist()
    if page > 1:
        with pytest.raises(ValueError):
            na.alloc(page + 1)


def test_engine_tokens_do_not_depend_on_the_implementation(tmp_path, monkeypatch):
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import write_tiny_qwen3_checkpoint
    path = write_tiny_qwen3_checkpoint(str(tmp_path / "m"))
    shared = list(range(5, 45))
    prompts = [shared + [60, 61, 62], shared + [70, 71], [9, 8, 7] * 9, shared[:20] + [80, 81, 82, 83]]
    sp = {"max_new_tokens": 10, "temperature": 0, "ignore_eos": True}

    def run():
        ps.reset_state()
        eng = Engine(model_path=path, device="cpu", dtype="float32", page_size=4, skip_tokenizer_init=True,
                     max_total_tokens=256, enable_single_process=True, chunked_prefill_size=16)
        try:
            kind = type(eng.scheduler.tree_cache).__name__, type(eng.scheduler.token_to_kv_pool_allocator).__name__
            a = [o["output_ids"] for o in eng.generate(input_ids=prompts, sampling_params=sp)]
            b = eng.generate(input_ids=prompts, sampling_params=sp)          # second pass hits the cache
            cached = [o["meta_info"]["cached_tokens"] for o in b]
            eng.scheduler.check_memory()
            return kind, a, [o["output_ids"] for o in b], cached
        finally:
            eng.shutdown()

    kind_n, a1, a2, cached_n = run()
    assert kind_n == ("NativeRadixCache", "NativePagedAllocator")
    monkeypatch.setenv("SGLB_DISABLE_NATIVE_SCHED", "1")
    kind_p, b1, b2, cached_p = run()
    assert kind_p == ("RadixCache", "PagedTokenToKVPoolAllocator")
    assert a1 == a2 == b1 == b2 and cached_n == cached_p and min(cached_n) > 0


def test_native_decode_step_builder_matches_python_arithmetic():
    """`PagedAllocator.build_decode_step` = last-slot gather + alloc_decode + table writes + page deltas."""
    import numpy as np
    from sglang_jax_b200.mem_cache import native as nat
    if not nat.available():
        import pytest
        pytest.skip("native scheduler structures not built")
    P = 4
    a = nat.NativePagedAllocator(64 * P, P)
    b = nat.NativePagedAllocator(64 * P, P)
    rng = np.random.RandomState(0)
    table_a = np.zeros((6, 40), np.int32)
    table_b = np.zeros((6, 40), np.int32)
    lens = np.array([3, 4, 8, 1, 9], np.int32)          # rows 1 and 2 sit on a page boundary
    rows = np.array([4, 0, 2, 5, 1], np.int32)
    for t, al in ((table_a, a), (table_b, b)):
        for r, n in zip(rows, lens):
            pre = np.zeros(1, np.int64)
            got = al.alloc_extend(pre, np.array([n], np.int64), np.array([-1], np.int64), int(n))
            t[r, :n] = got
    assert np.array_equal(table_a, table_b)
    # python statement of the step
    last = np.array([table_a[r, n - 1] for r, n in zip(rows, lens)], np.int32)
    want = a.alloc_decode(lens + 1, last)
    for r, n, loc in zip(rows, lens, want):
        table_a[r, n] = loc
    out, new_lens, positions, placeholders, d_rows, d_pos, d_ids = b.build_decode_step(table_b, rows, lens)
    assert np.array_equal(out, want) and np.array_equal(table_a, table_b)
    assert new_lens.tolist() == (lens + 1).tolist() and positions.tolist() == lens.tolist()
    assert placeholders.tolist() == (-(rows + 1)).tolist()
    assert d_rows.tolist() == [0, 2] and d_pos.tolist() == [1, 2] and d_ids.tolist() == [want[1] // P, want[2] // P]
    assert a.available_size() == b.available_size()
    # not enough pages: nothing changes
    small = nat.NativePagedAllocator(1 * P, P)
    t = np.zeros((2, 16), np.int32)
    t[0, :4] = small.alloc(4)
    before = t.copy()
    assert small.build_decode_step(t, np.array([0], np.int32), np.array([4], np.int32)) is None
    assert np.array_equal(t, before) and small.available_size() == 0
