"""Native (C++) paged allocator and radix-tree prefix cache behind the Python interfaces.

`csrc/sched/sched_native.cpp` owns the free list and the tree (token comparison, node splits, LRU
eviction); the classes here adapt it to `BaseTokenToKVPoolAllocator` / `RadixCache` so the
scheduler, the policies and the request hooks (`cache_finished_req`, `cache_unfinished_req`) are
the same code for both implementations.  `available()` is False when the extension has not been
built or `SGLB_DISABLE_NATIVE_SCHED=1`; the Python classes are used then."""

from __future__ import annotations

import os

import numpy as np

from .allocator import BaseTokenToKVPoolAllocator
from .base_prefix_cache import MatchResult
from .radix_cache import RadixCache, RadixKey

try:
    from . import _sched_native as _n
except ImportError:                      # not built: callers fall back to the Python structures
    _n = None


def available() -> bool:
    return _n is not None and not os.environ.get("SGLB_DISABLE_NATIVE_SCHED")


class NativePagedAllocator(BaseTokenToKVPoolAllocator):
    """Free list of pages 1..num_pages in C++ (`page_size == 1` = a free list of slots)."""

    def __init__(self, size: int, page_size: int, kvcache=None, dp_size: int = 1):
        super().__init__(size, page_size, kvcache, dp_size)
        self.num_pages = size // page_size
        self._a = _n.PagedAllocator(int(size), int(page_size))

    def clear(self):
        self._a.clear()
        self.is_not_in_free_group = True

    def available_size(self, dp_rank: int = 0) -> int:
        return self._a.available_size()

    def alloc(self, need_size: int, dp_rank: int = 0):
        return self._a.alloc(int(need_size))

    def alloc_extend(self, prefix_lens, seq_lens, last_loc, extend_num_tokens, dp_rank: int = 0):
        return self._a.alloc_extend(np.asarray(prefix_lens, np.int64), np.asarray(seq_lens, np.int64),
                                    np.asarray(last_loc, np.int64), int(extend_num_tokens))

    def alloc_decode(self, seq_lens, last_loc, dp_rank: int = 0):
        return self._a.alloc_decode(np.asarray(seq_lens, np.int64), np.asarray(last_loc, np.int64))

    def build_decode_step(self, req_to_token: np.ndarray, rows: np.ndarray, kv_lens: np.ndarray):
        """One decode step's slots, table writes and batch arrays in a single native call
        (`PagedAllocator::build_decode_step`); None when the pool lacks the pages (nothing changed)."""
        return self._a.build_decode_step(req_to_token, rows, kv_lens)

    def free(self, free_index, dp_rank: int = 0):
        self._a.free(np.asarray(free_index, np.int32).ravel())

    def free_group_begin(self):
        self.is_not_in_free_group = False
        self._a.free_group_begin()

    def free_group_end(self):
        self.is_not_in_free_group = True
        self._a.free_group_end()

    def backup_state(self):
        return self._a.backup_state()

    def restore_state(self, state):
        self._a.restore_state(np.asarray(state, np.int32))

    @property
    def free_pages(self):
        return self._a.backup_state()


class NodeRef:
    """Handle of a native tree node (what requests keep as `last_node`)."""
    __slots__ = ("tree", "id")

    def __init__(self, tree, node_id: int):
        self.tree, self.id = tree, node_id

    def __eq__(self, other):
        return isinstance(other, NodeRef) and other.id == self.id and other.tree is self.tree

    def __hash__(self):
        return hash(self.id)

    def _info(self):
        return self.tree.info(self.id)

    @property
    def children(self):
        return {c: NodeRef(self.tree, c) for c in self._info()[1]}

    @property
    def parent(self):
        p = self._info()[0]
        return None if p < 0 else NodeRef(self.tree, p)

    @property
    def lock_ref(self):
        return self._info()[2]

    @property
    def key(self):
        return self.tree.key_value(self.id)[0].tolist()

    @property
    def value(self):
        return self.tree.key_value(self.id)[1]

    @property
    def evicted(self):
        return not self.tree.alive(self.id)

    def __repr__(self):
        return f"NodeRef({self.id})"


class NativeRadixCache(RadixCache):
    def reset(self):
        self._t = _n.RadixTree(int(self.page_size))
        self.root_node = NodeRef(self._t, self._t.root_id())
        self._ns: dict = {}
        self._ns_rev: list = []

    def _ns_id(self, ns) -> int:
        i = self._ns.get(ns)
        if i is None:
            i = self._ns[ns] = len(self._ns_rev)
            self._ns_rev.append(ns)
        return i

    def _ids_for_dp(self, dp_rank):
        if dp_rank is None:
            return []
        ids = [i for i, ns in enumerate(self._ns_rev) if ns[1] == dp_rank]
        return ids or [-1]          # no namespace of that rank yet: match nothing

    def match_prefix(self, key: RadixKey, **kw) -> MatchResult:
        key = self._convert(key)
        if self.disable or len(key) == 0:
            return MatchResult(np.empty(0, np.int32), self.root_node, self.root_node)
        vals, nid = self._t.match(np.asarray(key.token_ids, np.int64), self._ns_id(key.namespace))
        node = NodeRef(self._t, nid)
        return MatchResult(vals, node, node)

    def insert(self, key: RadixKey, value=None, **kw) -> int:
        if self.disable:
            return 0
        key = self._convert(key)
        tokens = np.asarray(key.token_ids, np.int64)
        value = tokens.astype(np.int32) if value is None else np.asarray(value, np.int32)[: len(tokens)]
        existed, new_id, parent_id, n = self._t.insert(tokens[: len(value)], value, self._ns_id(key.namespace))
        if new_id >= 0 and self.enable_kv_cache_events:
            self.kv_event_queue.append({"type": "BlockStored", "node": new_id, "parent": parent_id, "num_tokens": n})
        return existed

    def evict(self, num_tokens: int, dp_rank: int | None = None):
        if self.disable or num_tokens <= 0:
            return 0
        freed = 0
        for ns, nid, vals in self._t.evict(int(num_tokens), self._ids_for_dp(dp_rank)):
            self.token_to_kv_pool_allocator.free(vals, dp_rank=self._ns_rev[ns][1] or 0)
            freed += len(vals)
            if self.enable_kv_cache_events:
                self.kv_event_queue.append({"type": "BlockRemoved", "node": nid})
        return freed

    def inc_lock_ref(self, node) -> int:
        if self.disable or node is None:
            return 0
        return self._t.inc_lock(node.id)

    def dec_lock_ref(self, node) -> int:
        if self.disable or node is None:
            return 0
        return self._t.dec_lock(node.id)

    def _sum(self, sizes: dict, dp_rank):
        return sum(v for i, v in sizes.items() if dp_rank is None or self._ns_rev[i][1] == dp_rank)

    def evictable_size(self, dp_rank: int | None = None) -> int:
        return self._sum(self._t.evictable(), dp_rank)

    def protected_size(self, dp_rank: int | None = None) -> int:
        return self._sum(self._t.protected_sizes(), dp_rank)

    def total_size(self) -> int:
        return self._t.total_size()

    def all_values_flatten(self) -> np.ndarray:
        return self._t.all_values()

    def pretty_print(self):
        lines = []

        def rec(node, depth):
            for c in node.children.values():
                k = c.key
                lines.append(" " * depth * 2 + f"[{len(k)}] {k[:8]}{'...' if len(k) > 8 else ''} lock={c.lock_ref}")
                rec(c, depth + 1)

        rec(self.root_node, 0)
        lines.append(f"#tokens: {self.total_size()}")
        print("\n".join(lines))
        return lines


def make_allocator(size: int, page_size: int, kvcache=None):
    """The scheduler's slot allocator: native when built, else the Python classes."""
    if available():
        return NativePagedAllocator(size, page_size, kvcache)
    from .allocator import PagedTokenToKVPoolAllocator, TokenToKVPoolAllocator
    return TokenToKVPoolAllocator(size, kvcache) if page_size == 1 else PagedTokenToKVPoolAllocator(size, page_size, kvcache)


def make_radix_cache(*args, **kw) -> RadixCache:
    return (NativeRadixCache if available() else RadixCache)(*args, **kw)
