"""Radix-tree prefix cache over KV slots.

Behavioural contract of the reference's `RadixCache`
(`python/sgl_jax/srt/mem_cache/radix_cache.py:154-641`):

* keys are token-id sequences namespaced by ``(extra_key, dp_rank)``;
* with ``page_size > 1`` everything is page granular: lookups truncate the key to
  a multiple of the page size, children are indexed by their first *page* of
  tokens and nodes only split on page boundaries;
* leaves that no running request locks are evicted least-recently-used first;
* ``cache_finished_req`` / ``cache_unfinished_req`` insert the page-aligned part
  of a request's tokens, free slots that duplicate an existing branch, and (for
  unfinished requests) rewrite the request's slot table to the canonical slots.

The implementation is this project's own: children live in one dict per node
keyed by ``(namespace, first-page tuple)`` at the root and ``first-page tuple``
below it, and eviction keeps per-namespace counters so `evictable_size(dp_rank)`
is O(1).
"""

from __future__ import annotations

import heapq
import time
from collections import defaultdict
from typing import Any

import numpy as np

from .base_prefix_cache import BasePrefixCache, MatchResult


class RadixKey:
    __slots__ = ("token_ids", "extra_key", "dp_rank")

    def __init__(self, token_ids, extra_key: str | None = None, dp_rank: int = 0):
        self.token_ids = token_ids if isinstance(token_ids, list) else list(token_ids)
        self.extra_key = extra_key
        self.dp_rank = dp_rank

    def __len__(self):
        return len(self.token_ids)

    def __getitem__(self, s):
        return RadixKey(self.token_ids[s], self.extra_key, self.dp_rank)

    @property
    def namespace(self):
        return (self.extra_key, self.dp_rank)

    def __repr__(self):
        return f"RadixKey(ns={self.namespace}, n={len(self.token_ids)})"


class TreeNode:
    _counter = 0
    __slots__ = ("children", "parent", "key", "value", "lock_ref", "last_access_time",
                 "hit_count", "id", "namespace", "host_value", "child_key", "loading")

    def __init__(self):
        self.children: dict[Any, TreeNode] = {}
        self.parent: TreeNode | None = None
        self.key: list[int] = []
        self.value: np.ndarray | None = None
        self.lock_ref = 0
        self.last_access_time = time.monotonic()
        self.hit_count = 0
        self.namespace = None
        self.host_value = None
        self.child_key = None
        self.loading = False
        TreeNode._counter += 1
        self.id = TreeNode._counter

    @property
    def evicted(self):
        return self.value is None

    @property
    def backuped(self):
        return self.host_value is not None

    def __lt__(self, other):
        return self.last_access_time < other.last_access_time


def _match_len(a: list[int], b: list[int], page: int) -> int:
    n = min(len(a), len(b))
    if page == 1:
        i = 0
        while i < n and a[i] == b[i]:
            i += 1
        return i
    i = 0
    while i + page <= n and a[i:i + page] == b[i:i + page]:
        i += page
    return i


class RadixCache(BasePrefixCache):
    def __init__(self, req_to_token_pool, token_to_kv_pool_allocator, page_size: int = 1,
                 disable: bool = False, enable_kv_cache_events: bool = False, is_eagle: bool = False):
        self.req_to_token_pool = req_to_token_pool
        self.token_to_kv_pool_allocator = token_to_kv_pool_allocator
        self.page_size = page_size
        self.disable = disable
        self.enable_kv_cache_events = enable_kv_cache_events
        self.is_eagle = is_eagle
        self.kv_event_queue: list = []
        self.reset()

    # ---------------------------------------------------------------- basic
    def reset(self):
        self.root_node = TreeNode()
        self.root_node.key = []
        self.root_node.value = np.empty(0, np.int32)
        self.root_node.lock_ref = 1
        self._evictable = defaultdict(int)
        self._protected = defaultdict(int)

    def _child_key(self, tokens: list[int], ns, at_root: bool):
        head = tokens[0] if self.page_size == 1 else tuple(tokens[:self.page_size])
        return (ns, head) if at_root else head

    def _convert(self, key: RadixKey) -> RadixKey:
        """EAGLE drafts are keyed by bigrams (token i, token i+1)."""
        if not self.is_eagle:
            return key
        t = key.token_ids
        return RadixKey([t[i] * 1_000_003 + t[i + 1] for i in range(len(t) - 1)], key.extra_key, key.dp_rank)

    def _page_trunc(self, n: int) -> int:
        return n // self.page_size * self.page_size

    # ---------------------------------------------------------------- match
    def match_prefix(self, key: RadixKey, **kw) -> MatchResult:
        key = self._convert(key)
        if self.disable or len(key) == 0:
            return MatchResult(np.empty(0, np.int32), self.root_node, self.root_node)
        tokens = key.token_ids[: self._page_trunc(len(key))]
        if not tokens:
            return MatchResult(np.empty(0, np.int32), self.root_node, self.root_node)
        values, node = self._match(tokens, key.namespace)
        out = np.concatenate(values) if values else np.empty(0, np.int32)
        return MatchResult(out, node, node)

    def _match(self, tokens: list[int], ns):
        node = self.root_node
        now = time.monotonic()
        node.last_access_time = now
        values = []
        pos = 0
        while pos < len(tokens):
            ck = self._child_key(tokens[pos:], ns, node is self.root_node)
            child = node.children.get(ck)
            if child is None or child.evicted:
                break
            child.last_access_time = now
            m = _match_len(child.key, tokens[pos:], self.page_size)
            if m < len(child.key):
                if m == 0:
                    break
                child = self._split(child, m)
                values.append(child.value)
                node = child
                break
            values.append(child.value)
            node = child
            pos += m
        return values, node

    def _split(self, child: TreeNode, m: int) -> TreeNode:
        """Cut `child` at `m` tokens; returns the new upper node."""
        parent = child.parent
        upper = TreeNode()
        upper.namespace = child.namespace
        upper.parent = parent
        upper.key = child.key[:m]
        upper.value = child.value[:m]
        upper.lock_ref = child.lock_ref
        upper.last_access_time = child.last_access_time
        upper.child_key = child.child_key
        parent.children[child.child_key] = upper
        child.parent = upper
        child.key = child.key[m:]
        child.value = child.value[m:]
        child.child_key = self._child_key(child.key, child.namespace, False)
        upper.children[child.child_key] = child
        return upper

    # ---------------------------------------------------------------- insert
    def insert(self, key: RadixKey, value=None, **kw) -> int:
        """Insert ``key -> value``; returns how many leading tokens already existed."""
        if self.disable:
            return 0
        key = self._convert(key)
        tokens = key.token_ids
        if value is None:
            value = np.asarray(tokens, dtype=np.int32)
        value = np.asarray(value, dtype=np.int32)[: len(tokens)]
        n = self._page_trunc(len(tokens))
        tokens, value = tokens[:n], value[:n]
        if n == 0:
            return 0
        ns = key.namespace
        node = self.root_node
        now = time.monotonic()
        pos = 0
        existed = 0
        while pos < n:
            ck = self._child_key(tokens[pos:], ns, node is self.root_node)
            child = node.children.get(ck)
            if child is None:
                break
            child.last_access_time = now
            m = _match_len(child.key, tokens[pos:], self.page_size)
            if m == 0:
                break
            if m < len(child.key):
                child = self._split(child, m)
            if child.evicted:
                # a host-only node regains device slots
                child.value = value[pos:pos + m].copy()
                self._evictable[ns] += m
            else:
                existed += m
            node = child
            pos += m
        if pos < n:
            new = TreeNode()
            new.namespace = ns
            new.parent = node
            new.key = tokens[pos:]
            new.value = value[pos:].copy()
            new.child_key = self._child_key(new.key, ns, node is self.root_node)
            node.children[new.child_key] = new
            self._evictable[ns] += len(new.key)
            self._record_store(new)
        return existed

    # ---------------------------------------------------------------- request hooks
    def cache_finished_req(self, req, is_insert: bool = True, **kw):
        """Move a finished request's KV into the tree (or free it) and release its row."""
        pool = self.req_to_token_pool
        alloc = self.token_to_kv_pool_allocator
        kv_len = req.committed_kv_len()
        kv_indices = pool.read(req.req_pool_idx, kv_len).copy()
        dp = getattr(req, "dp_rank", 0) or 0
        if self.disable:
            alloc.free(kv_indices, dp_rank=dp)
            return
        if not is_insert:
            # the matched prefix belongs to the tree; only the request's own slots go back
            alloc.free(kv_indices[req.last_matched_prefix_len:], dp_rank=dp)
            self.dec_lock_ref(req.last_node)
            return
        token_ids = (req.origin_input_ids + req.output_ids)[:kv_len]
        key = RadixKey(token_ids, req.extra_key, dp)
        if self.is_eagle:
            kv_len_eff = max(kv_len - 1, 0)
        else:
            kv_len_eff = kv_len
        aligned = self._page_trunc(kv_len_eff)
        # leading slots that already belong to the tree (everything after is the request's own)
        old_prefix_len = req.last_matched_prefix_len
        new_prefix_len = self.insert(key[:aligned + (1 if self.is_eagle else 0)], kv_indices[:aligned])
        # slots duplicated by an already cached branch
        alloc.free(kv_indices[old_prefix_len:new_prefix_len], dp_rank=dp)
        # unaligned tail is never shared
        alloc.free(kv_indices[aligned:], dp_rank=dp)
        self.dec_lock_ref(req.last_node)

    def cache_unfinished_req(self, req, chunked: bool = False, **kw):
        """After a prefill chunk: publish the aligned prefix and re-point the request at
        the canonical slots so later requests can share it."""
        if self.disable:
            kv_len = len(req.fill_ids)
            req.prefix_indices = self.req_to_token_pool.read(req.req_pool_idx, kv_len).copy()
            return
        pool = self.req_to_token_pool
        alloc = self.token_to_kv_pool_allocator
        dp = getattr(req, "dp_rank", 0) or 0
        token_ids = req.fill_ids
        kv_len = len(token_ids)
        kv_indices = pool.read(req.req_pool_idx, kv_len).copy()
        kv_len_eff = kv_len - 1 if self.is_eagle else kv_len
        aligned = self._page_trunc(kv_len_eff)
        key = RadixKey(token_ids, req.extra_key, dp)
        # leading slots that already belong to the tree (everything after is the request's own)
        old_prefix_len = req.last_matched_prefix_len
        new_prefix_len = self.insert(key[:aligned + (1 if self.is_eagle else 0)], kv_indices[:aligned])
        alloc.free(kv_indices[old_prefix_len:new_prefix_len], dp_rank=dp)
        res = self.match_prefix(key[:aligned + (1 if self.is_eagle else 0)])
        new_indices, new_last = res.device_indices, res.last_device_node
        assert len(new_indices) >= old_prefix_len or self.is_eagle, (len(new_indices), old_prefix_len)
        if len(new_indices) > old_prefix_len:
            pool.write(req.req_pool_idx, old_prefix_len, new_indices[old_prefix_len:])
        self.dec_lock_ref(req.last_node)
        self.inc_lock_ref(new_last)
        req.last_node = new_last
        if len(new_indices) < kv_len:
            req.prefix_indices = np.concatenate([new_indices, kv_indices[len(new_indices):]])
        else:
            req.prefix_indices = new_indices
        req.last_matched_prefix_len = len(new_indices)

    # ---------------------------------------------------------------- eviction / locks
    def _leaves(self, ns_filter=None):
        out = []
        stack = [self.root_node]
        while stack:
            n = stack.pop()
            live_children = [c for c in n.children.values() if not c.evicted]
            if n is not self.root_node and not n.evicted and not live_children:
                if ns_filter is None or n.namespace[1] == ns_filter:
                    out.append(n)
            stack.extend(n.children.values())
        return out

    def evict(self, num_tokens: int, dp_rank: int | None = None):
        if self.disable or num_tokens <= 0:
            return 0
        leaves = [n for n in self._leaves(dp_rank) if n.lock_ref == 0]
        heapq.heapify(leaves)
        freed = 0
        while freed < num_tokens and leaves:
            n = heapq.heappop(leaves)
            if n.lock_ref > 0 or n.evicted:
                continue
            self.token_to_kv_pool_allocator.free(n.value, dp_rank=n.namespace[1] or 0)
            freed += len(n.value)
            self._evictable[n.namespace] -= len(n.value)
            self._record_remove(n)
            self._drop(n)
            p = n.parent
            if p is not self.root_node and p.lock_ref == 0 and not p.evicted and \
                    not any(not c.evicted for c in p.children.values()):
                heapq.heappush(leaves, p)
        return freed

    def _drop(self, n: TreeNode):
        if n.backuped:
            n.value = None  # keep as host-only node
        else:
            del n.parent.children[n.child_key]

    def inc_lock_ref(self, node: TreeNode) -> int:
        if self.disable or node is None:
            return 0
        delta = 0
        while node is not self.root_node and node is not None:
            if node.lock_ref == 0 and not node.evicted:
                n = len(node.value)
                self._evictable[node.namespace] -= n
                self._protected[node.namespace] += n
                delta -= n
            node.lock_ref += 1
            node = node.parent
        return delta

    def dec_lock_ref(self, node: TreeNode) -> int:
        if self.disable or node is None:
            return 0
        delta = 0
        while node is not self.root_node and node is not None:
            if node.lock_ref == 1 and not node.evicted:
                n = len(node.value)
                self._evictable[node.namespace] += n
                self._protected[node.namespace] -= n
                delta += n
            node.lock_ref -= 1
            assert node.lock_ref >= 0
            node = node.parent
        return delta

    def evictable_size(self, dp_rank: int | None = None) -> int:
        return sum(v for (ek, dp), v in self._evictable.items() if dp_rank is None or dp == dp_rank)

    def protected_size(self, dp_rank: int | None = None) -> int:
        return sum(v for (ek, dp), v in self._protected.items() if dp_rank is None or dp == dp_rank)

    def total_size(self) -> int:
        total = 0
        stack = [self.root_node]
        while stack:
            n = stack.pop()
            if n is not self.root_node and not n.evicted:
                total += len(n.value)
            stack.extend(n.children.values())
        return total

    def all_values_flatten(self) -> np.ndarray:
        vals = []
        stack = [self.root_node]
        while stack:
            n = stack.pop()
            if n is not self.root_node and not n.evicted:
                vals.append(n.value)
            stack.extend(n.children.values())
        return np.concatenate(vals) if vals else np.empty(0, np.int32)

    def pretty_print(self):
        lines = []

        def rec(n, depth):
            for c in n.children.values():
                lines.append(" " * depth * 2 + f"[{len(c.key)}] {c.key[:8]}{'...' if len(c.key) > 8 else ''} "
                             f"lock={c.lock_ref} ns={c.namespace}{' (host)' if c.evicted else ''}")
                rec(c, depth + 1)

        rec(self.root_node, 0)
        lines.append(f"#tokens: {self.total_size()}")
        print("\n".join(lines))
        return lines

    # ---------------------------------------------------------------- KV events
    def _record_store(self, node):
        if self.enable_kv_cache_events:
            self.kv_event_queue.append({"type": "BlockStored", "node": node.id,
                                        "parent": node.parent.id if node.parent else None,
                                        "num_tokens": len(node.key)})

    def _record_remove(self, node):
        if self.enable_kv_cache_events:
            self.kv_event_queue.append({"type": "BlockRemoved", "node": node.id})

    def take_events(self):
        ev, self.kv_event_queue = self.kv_event_queue, []
        return ev
