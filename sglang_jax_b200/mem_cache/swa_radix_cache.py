"""Radix cache for hybrid sliding-window models.

Reference: `python/sgl_jax/srt/mem_cache/swa_radix_cache.py:290` (`evict` :509,
`evict_req_swa` :760).

Every cached token owns a slot in the full-attention pool and one in the (smaller)
sliding-window pool.  Window layers only ever read the last `sliding_window` tokens, so
the SWA slots of older tokens can be given back while the full-attention slots stay
cached.  A node whose SWA slots were released is a *tombstone*: it still extends a prefix
for the full-attention layers, but a match may only end at a point that has at least
`sliding_window` tokens of live SWA KV directly before it (or reaches back to the root
without meeting a tombstone).

Two orders of eviction exist: full (drops leaves entirely) and SWA (tombstones internal
nodes, drops leaves), each least-recently-used first; two lock counts protect a running
request's path (`full_lock_ref` on the whole path, `swa_lock_ref` on the part inside the
window).
"""

from __future__ import annotations

import heapq
import time
from collections import defaultdict
from typing import Any

import numpy as np

from .base_prefix_cache import BasePrefixCache, MatchResult
from .radix_cache import RadixKey, _match_len


class SWATreeNode:
    _counter = 0

    def __init__(self):
        self.children: dict[Any, SWATreeNode] = {}
        self.parent: SWATreeNode | None = None
        self.key: list[int] = []
        self.value: np.ndarray | None = None       # full-pool slots
        self.swa_tombstone = False
        self.full_lock_ref = 0
        self.swa_lock_ref = 0
        self.last_access_time = time.monotonic()
        self.namespace = None
        self.child_key = None
        self.swa_uuid: int | None = None
        self.lock_uuids: list = []          # SWA lock boundaries of the locks taken on this node
        SWATreeNode._counter += 1
        self.id = SWATreeNode._counter

    def __lt__(self, other):
        return self.last_access_time < other.last_access_time


class SWARadixCache(BasePrefixCache):
    def __init__(self, req_to_token_pool, token_to_kv_pool_allocator, sliding_window_size: int, page_size: int = 1,
                 disable: bool = False):
        self.req_to_token_pool = req_to_token_pool
        self.token_to_kv_pool_allocator = token_to_kv_pool_allocator
        self.sliding_window_size = int(sliding_window_size)
        self.page_size = page_size
        self.disable = disable
        self._uuid = 0
        self.reset()

    # ------------------------------------------------------------------ basics
    def reset(self):
        self.root_node = SWATreeNode()
        self.root_node.full_lock_ref = 1
        self.root_node.swa_lock_ref = 1
        self.full_evictable = 0
        self.swa_evictable = 0
        self.full_protected = 0
        self.swa_protected = 0

    def _child_key(self, tokens, ns, at_root):
        head = tokens[0] if self.page_size == 1 else tuple(tokens[: self.page_size])
        return (ns, head) if at_root else head

    def _trunc(self, n):
        return n // self.page_size * self.page_size

    def _next_uuid(self):
        self._uuid += 1
        return self._uuid

    # ------------------------------------------------------------------ match
    def match_prefix(self, key: RadixKey, **kw) -> MatchResult:
        empty = MatchResult(np.empty(0, np.int32), self.root_node, self.root_node)
        if self.disable or len(key) == 0:
            return empty
        tokens = key.token_ids[: self._trunc(len(key))]
        if not tokens:
            return empty
        ns = key.namespace
        node = self.root_node
        now = time.monotonic()
        values: list[np.ndarray] = []
        # the best end point so far: (number of value chunks, node)
        best_n, best_node = 0, self.root_node
        live_run = float("inf")       # tokens of live SWA KV directly before the current point
        pos = 0
        while pos < len(tokens):
            child = node.children.get(self._child_key(tokens[pos:], ns, node is self.root_node))
            if child is None:
                break
            m = _match_len(child.key, tokens[pos:], self.page_size)
            if m == 0:
                break
            if m < len(child.key):
                child = self._split(child, m)
            child.last_access_time = now
            if child.swa_tombstone:
                live_run = 0
            else:
                live_run = live_run + m
            values.append(child.value)
            node = child
            pos += m
            if live_run >= self.sliding_window_size:
                best_n, best_node = len(values), node
        out = np.concatenate(values[:best_n]) if best_n else np.empty(0, np.int32)
        return MatchResult(out, best_node, best_node)

    def _split(self, child: SWATreeNode, m: int) -> SWATreeNode:
        parent = child.parent
        upper = SWATreeNode()
        upper.namespace = child.namespace
        upper.parent = parent
        upper.key = child.key[:m]
        upper.value = child.value[:m]
        upper.swa_tombstone = child.swa_tombstone
        upper.full_lock_ref = child.full_lock_ref
        upper.swa_lock_ref = child.swa_lock_ref
        upper.swa_uuid = child.swa_uuid
        child.swa_uuid = None
        upper.last_access_time = child.last_access_time
        upper.child_key = child.child_key
        parent.children[child.child_key] = upper
        child.parent = upper
        child.key = child.key[m:]
        child.value = child.value[m:]
        child.child_key = self._child_key(child.key, child.namespace, False)
        upper.children[child.child_key] = child
        return upper

    # ------------------------------------------------------------------ insert
    def insert(self, key: RadixKey, value=None, prev_prefix_len: int = 0, swa_evicted_seqlen: int = 0, **kw) -> int:
        """Returns how many tokens already existed (`self.last_dup_ranges` lists them as
        `(start, end)`).  Tombstones on the path that lie beyond `prev_prefix_len` (the request
        did not reuse them, so it computed fresh SWA KV there) are revived with the request's
        slots; tokens before `swa_evicted_seqlen` have lost their SWA KV already and enter
        the tree as tombstones."""
        self.last_dup_ranges: list[tuple[int, int]] = []
        if self.disable:
            return 0
        tokens = key.token_ids
        value = np.asarray(value if value is not None else tokens, dtype=np.int32)[: len(tokens)]
        n = self._trunc(len(tokens))
        tokens, value = tokens[:n], value[:n]
        if n == 0:
            return 0
        ns = key.namespace
        node = self.root_node
        now = time.monotonic()
        pos = existed = 0
        alloc = self.token_to_kv_pool_allocator
        while pos < n:
            child = node.children.get(self._child_key(tokens[pos:], ns, node is self.root_node))
            if child is None:
                break
            m = _match_len(child.key, tokens[pos:], self.page_size)
            if m == 0:
                break
            if m < len(child.key):
                child = self._split(child, m)
            child.last_access_time = now
            if child.swa_tombstone and pos >= prev_prefix_len and pos >= swa_evicted_seqlen \
                    and child.full_lock_ref == 0:
                # swap in the request's slots (they carry live SWA KV); the old full slots go back
                full = getattr(alloc, "full_attn_allocator", alloc)
                full.free(child.value)
                child.value = value[pos:pos + m].copy()
                child.swa_tombstone = False
                self.swa_evictable += m
            else:
                existed += m
                self.last_dup_ranges.append((pos, pos + m))
            node = child
            pos += m
        cut = min(self._trunc(swa_evicted_seqlen), n)
        for lo, hi, dead in ((pos, max(cut, pos), True), (max(cut, pos), n, False)):
            if hi <= lo:
                continue
            new = SWATreeNode()
            new.namespace = ns
            new.parent = node
            new.key = tokens[lo:hi]
            new.value = value[lo:hi].copy()
            new.swa_tombstone = dead
            new.child_key = self._child_key(new.key, ns, node is self.root_node)
            node.children[new.child_key] = new
            self.full_evictable += hi - lo
            if not dead:
                self.swa_evictable += hi - lo
            node = new
        return existed

    # ------------------------------------------------------------------ request hooks
    def cache_finished_req(self, req, is_insert: bool = True, **kw):
        pool, alloc = self.req_to_token_pool, self.token_to_kv_pool_allocator
        kv_len = req.committed_kv_len()
        kv_indices = pool.read(req.req_pool_idx, kv_len).copy()
        if self.disable:
            alloc.free(kv_indices)
            return
        old_prefix = req.last_matched_prefix_len
        if not is_insert:
            alloc.free(kv_indices[old_prefix:])
            self.dec_lock_ref(req.last_node, getattr(req, "swa_uuid_for_lock", None))
            return
        aligned = self._trunc(kv_len)
        tokens = (req.origin_input_ids + req.output_ids)[:aligned]
        self.insert(RadixKey(tokens, req.extra_key, getattr(req, "dp_rank", 0) or 0), kv_indices[:aligned],
                    prev_prefix_len=old_prefix, swa_evicted_seqlen=getattr(req, "swa_evicted_seqlen", 0))
        for lo, hi in self.last_dup_ranges:
            lo = max(lo, old_prefix)      # the matched prefix is the tree's own
            if hi > lo:
                alloc.free(kv_indices[lo:hi])
        alloc.free(kv_indices[aligned:])
        self.dec_lock_ref(req.last_node, getattr(req, "swa_uuid_for_lock", None))

    def cache_unfinished_req(self, req, chunked: bool = False, **kw):
        pool, alloc = self.req_to_token_pool, self.token_to_kv_pool_allocator
        tokens = req.fill_ids
        kv_len = len(tokens)
        kv_indices = pool.read(req.req_pool_idx, kv_len).copy()
        if self.disable:
            req.prefix_indices = kv_indices
            return
        aligned = self._trunc(kv_len)
        old_prefix = req.last_matched_prefix_len
        dp = getattr(req, "dp_rank", 0) or 0
        key = RadixKey(tokens[:aligned], req.extra_key, dp)
        self.insert(key, kv_indices[:aligned], prev_prefix_len=old_prefix)
        for lo, hi in self.last_dup_ranges:
            lo = max(lo, old_prefix)
            if hi > lo:
                alloc.free(kv_indices[lo:hi])
        res = self.match_prefix(key)
        new_indices, new_last = res.device_indices, res.last_device_node
        if len(new_indices) > old_prefix:
            pool.write(req.req_pool_idx, old_prefix, new_indices[old_prefix:])
        self.dec_lock_ref(req.last_node, getattr(req, "swa_uuid_for_lock", None))
        req.swa_uuid_for_lock = self.inc_lock_ref(new_last)
        req.last_node = new_last
        if len(new_indices) < kv_len:
            req.prefix_indices = np.concatenate([new_indices, kv_indices[len(new_indices):]])
        else:
            req.prefix_indices = new_indices
        req.last_matched_prefix_len = len(new_indices)

    # ------------------------------------------------------------------ locks
    def inc_lock_ref(self, node: SWATreeNode):
        """Locks the whole path for full attention and its last `sliding_window` tokens for
        the window layers.  Returns the id that `dec_lock_ref` needs to undo the SWA part."""
        if self.disable or node is None:
            return None
        swa_locked = 0
        swa_uuid = None
        n = node
        while n is not self.root_node and n is not None:
            if n.full_lock_ref == 0:
                self.full_evictable -= len(n.key)
                self.full_protected += len(n.key)
            n.full_lock_ref += 1
            if swa_locked < self.sliding_window_size and not n.swa_tombstone:
                if n.swa_lock_ref == 0:
                    self.swa_evictable -= len(n.key)
                    self.swa_protected += len(n.key)
                n.swa_lock_ref += 1
                swa_locked += len(n.key)
                if swa_locked >= self.sliding_window_size:
                    if n.swa_uuid is None:
                        n.swa_uuid = self._next_uuid()
                    swa_uuid = n.swa_uuid
            n = n.parent
        node.lock_uuids.append(swa_uuid)
        return swa_uuid

    def dec_lock_ref(self, node: SWATreeNode, swa_uuid_for_lock=None):
        if self.disable or node is None:
            return
        if node.lock_uuids:
            # callers that do not carry the boundary id get the one recorded at lock time
            recorded = node.lock_uuids.pop()
            if swa_uuid_for_lock is None:
                swa_uuid_for_lock = recorded
        dec_swa = True
        n = node
        while n is not self.root_node and n is not None:
            if n.full_lock_ref == 1:
                self.full_evictable += len(n.key)
                self.full_protected -= len(n.key)
            n.full_lock_ref -= 1
            assert n.full_lock_ref >= 0
            if dec_swa and not n.swa_tombstone and n.swa_lock_ref > 0:
                if n.swa_lock_ref == 1:
                    self.swa_evictable += len(n.key)
                    self.swa_protected -= len(n.key)
                n.swa_lock_ref -= 1
                if swa_uuid_for_lock is not None and n.swa_uuid == swa_uuid_for_lock:
                    dec_swa = False
            n = n.parent

    # ------------------------------------------------------------------ eviction
    def _all_nodes(self):
        out, stack = [], [self.root_node]
        while stack:
            n = stack.pop()
            if n is not self.root_node:
                out.append(n)
            stack.extend(n.children.values())
        return out

    def _remove_leaf(self, n: SWATreeNode):
        alloc = self.token_to_kv_pool_allocator
        if n.swa_tombstone:
            alloc.full_attn_allocator.free(n.value) if hasattr(alloc, "full_attn_allocator") else alloc.free(n.value)
        else:
            alloc.free(n.value)
            self.swa_evictable -= len(n.key)
        self.full_evictable -= len(n.key)
        del n.parent.children[n.child_key]

    def evict(self, full_num_tokens: int = 0, swa_num_tokens: int = 0, dp_rank=None):
        """Returns `(full tokens freed, swa tokens freed)`."""
        if self.disable:
            return 0, 0
        full_freed = swa_freed = 0
        if full_num_tokens > 0:
            leaves = [n for n in self._all_nodes() if not n.children and n.full_lock_ref == 0]
            heapq.heapify(leaves)
            while full_freed < full_num_tokens and leaves:
                n = heapq.heappop(leaves)
                if n.children or n.full_lock_ref > 0 or n.parent is None or n.child_key not in n.parent.children:
                    continue
                full_freed += len(n.key)
                if not n.swa_tombstone:
                    swa_freed += len(n.key)
                p = n.parent
                self._remove_leaf(n)
                if p is not self.root_node and not p.children and p.full_lock_ref == 0:
                    heapq.heappush(leaves, p)
        if swa_freed < swa_num_tokens:
            cands = [n for n in self._all_nodes() if not n.swa_tombstone and n.swa_lock_ref == 0]
            heapq.heapify(cands)
            alloc = self.token_to_kv_pool_allocator
            while swa_freed < swa_num_tokens and cands:
                n = heapq.heappop(cands)
                if n.swa_tombstone or n.swa_lock_ref > 0 or n.parent is None or n.child_key not in n.parent.children:
                    continue
                if not n.children:
                    if n.full_lock_ref > 0:
                        continue
                    swa_freed += len(n.key)
                    full_freed += len(n.key)
                    p = n.parent
                    self._remove_leaf(n)
                    # a tombstone that lost its last child serves nobody: drop the chain upwards
                    while p is not self.root_node and not p.children and p.full_lock_ref == 0 and p.swa_tombstone:
                        full_freed += len(p.key)
                        pp = p.parent
                        self._remove_leaf(p)
                        p = pp
                else:
                    alloc.free_swa(n.value)
                    n.swa_tombstone = True
                    self.swa_evictable -= len(n.key)
                    swa_freed += len(n.key)
        return full_freed, swa_freed

    def evict_req_swa(self, req, pre_len: int) -> int:
        """Release the SWA slots a running request no longer needs: everything before
        `pre_len - sliding_window` (page aligned) that the tree does not own.  Returns the new
        `swa_evicted_seqlen`."""
        new_upto = self._trunc(max(pre_len - self.sliding_window_size, 0))
        start = max(getattr(req, "swa_evicted_seqlen", 0), req.last_matched_prefix_len)
        if new_upto > start:
            idx = self.req_to_token_pool.read(req.req_pool_idx, new_upto)[start:new_upto].copy()
            self.token_to_kv_pool_allocator.free_swa(idx)
            req.swa_evicted_seqlen = new_upto
        return getattr(req, "swa_evicted_seqlen", 0)

    # ------------------------------------------------------------------ sizes
    def evictable_size(self, dp_rank=None):
        return self.full_evictable

    def full_evictable_size(self):
        return self.full_evictable

    def swa_evictable_size(self):
        return self.swa_evictable

    def protected_size(self, dp_rank=None):
        return self.full_protected

    def full_protected_size(self):
        return self.full_protected

    def swa_protected_size(self):
        return self.swa_protected

    def total_size(self):
        full = sum(len(n.key) for n in self._all_nodes())
        swa = sum(len(n.key) for n in self._all_nodes() if not n.swa_tombstone)
        return full, swa

    def all_values_flatten(self):
        vals = [n.value for n in self._all_nodes()]
        return np.concatenate(vals) if vals else np.empty(0, np.int32)

    def pretty_print(self):
        def rec(n, d):
            for c in n.children.values():
                print(" " * d, len(c.key), c.key[:8], "T" if c.swa_tombstone else "-",
                      f"full_lock={c.full_lock_ref} swa_lock={c.swa_lock_ref}")
                rec(c, d + 2)
        rec(self.root_node, 0)
