"""Radix cache with a host-memory second tier (HiCache).

Reference: the HiCache hooks of `python/sgl_jax/srt/mem_cache/unified_radix_cache.py`
(`write_backup` :835, `evict_host` :1022, `init_load_back` :1061) and
`hicache_controller.py`.

A node may hold device slots (`value`), host pages (`host_value`) or both.
* write policies: `write_through` backs a node up the first time it is inserted or hit,
  `write_through_selective` after `threshold` hits, `write_back` only when it is evicted
  from the device;
* evicting a backed-up node from the device keeps it in the tree as a host-only node;
* `match_prefix` keeps walking through host-only nodes and reports `host_hit_length`;
  `init_load_back` gives those nodes device slots again and starts the host -> device copy;
* nodes are locked while a copy that involves them is in flight.
"""

from __future__ import annotations

import heapq
import logging
import time

import numpy as np

from .base_prefix_cache import MatchResult
from .hicache_controller import HiCacheController
from .host_kv_pool import LRUHostKVPool
from .radix_cache import RadixCache, RadixKey, TreeNode, _match_len

logger = logging.getLogger(__name__)


class HiRadixCache(RadixCache):
    def __init__(self, req_to_token_pool, token_to_kv_pool_allocator, page_size, device_pool,
                 hicache_ratio: float = 2.0, write_policy: str = "write_through", write_through_threshold: int = 1,
                 host_pages: int | None = None, **kw):
        super().__init__(req_to_token_pool, token_to_kv_pool_allocator, page_size, **kw)
        dev_pages = device_pool.size // page_size
        n_host = host_pages if host_pages is not None else max(int(dev_pages * hicache_ratio), 1)
        self.host_pool = LRUHostKVPool(device_pool, n_host)
        self.controller = HiCacheController(self.host_pool, write_policy)
        self.write_policy = write_policy
        self.write_threshold = 1 if write_policy == "write_through" else max(int(write_through_threshold), 1)
        self.ongoing_write: dict[int, tuple[TreeNode, np.ndarray]] = {}
        self.ongoing_load: dict[int, list[TreeNode]] = {}
        self._ticket_seq = 0
        logger.info("HiCache: %d host pages (%.2f GB), policy %s", n_host, self.host_pool.size_bytes() / 2 ** 30,
                    write_policy)

    def reset(self):
        super().reset()
        if hasattr(self, "controller"):
            self.controller.drain()
            self.ongoing_write.clear()
            self.ongoing_load.clear()
            self.host_pool.free_pages.clear()
            self.host_pool.free_pages.extend(range(self.host_pool.num_pages))

    # ------------------------------------------------------------------ pages of a node
    def _dev_pages(self, node: TreeNode) -> np.ndarray:
        return (node.value[:: self.page_size] // self.page_size).astype(np.int64)

    def _split(self, child: TreeNode, m: int) -> TreeNode:
        host = child.host_value
        dev_evicted = child.evicted
        if dev_evicted:
            # base split slices `value`; give it a placeholder and restore afterwards
            child.value = np.zeros(len(child.key), np.int32)
        upper = super()._split(child, m)
        if dev_evicted:
            upper.value = None
            child.value = None
        if host is not None:
            pm = m // self.page_size
            upper.host_value = host[:pm]
            child.host_value = host[pm:]
        return upper

    # ------------------------------------------------------------------ backup
    def inc_hit_count(self, node: TreeNode):
        if node is self.root_node or node.evicted or self.write_policy == "write_back":
            return
        node.hit_count += 1
        if node.hit_count >= self.write_threshold and not node.backuped and node.id not in self._writing_ids():
            self.write_backup(node)

    def _writing_ids(self):
        return {n.id for n, _ in self.ongoing_write.values()}

    def write_backup(self, node: TreeNode, blocking: bool = False) -> bool:
        n_pages = len(node.key) // self.page_size
        if n_pages == 0:
            return False
        host = self.host_pool.alloc(n_pages)
        if host is None:
            self.evict_host(n_pages)
            host = self.host_pool.alloc(n_pages)
            if host is None:
                return False
        t = self.controller.write(node.id, self._dev_pages(node), host)
        self._ticket_seq += 1
        self.ongoing_write[id(t)] = (node, host)
        self.inc_lock_ref(node)
        if blocking:
            self.controller.sync()
            self.check_hicache_events()
        return True

    def check_hicache_events(self):
        """Retire finished copies: a written node becomes backed up, loaded nodes unlock."""
        for t in self.controller.poll():
            if t.kind == "write":
                node, host = self.ongoing_write.pop(id(t))
                # the node may have been split while the copy ran: hand the pages out bottom-up
                n, rest = node, host
                while len(rest):
                    k = len(n.key) // self.page_size
                    n.host_value = rest[len(rest) - k:]
                    rest = rest[:len(rest) - k]
                    n = n.parent
                self.dec_lock_ref(node)
            else:
                for node in self.ongoing_load.pop(id(t), []):
                    self.dec_lock_ref(node)

    def ready_to_load_host_cache(self) -> int:
        return self.controller.wait_loads()

    # ------------------------------------------------------------------ insert / match
    def insert(self, key: RadixKey, value=None, **kw) -> int:
        existed = super().insert(key, value, **kw)
        if not self.disable and self.write_policy != "write_back":
            ckey = self._convert(key)
            n = self._page_trunc(len(ckey))
            node = self.root_node
            pos = 0
            tokens = ckey.token_ids[:n]
            while pos < n:
                ck = self._child_key(tokens[pos:], ckey.namespace, node is self.root_node)
                child = node.children.get(ck)
                if child is None:
                    break
                m = _match_len(child.key, tokens[pos:], self.page_size)
                if m < len(child.key):
                    break
                self.inc_hit_count(child)
                node = child
                pos += m
        return existed

    def match_prefix(self, key: RadixKey, **kw) -> MatchResult:
        key = self._convert(key)
        empty = MatchResult(np.empty(0, np.int32), self.root_node, self.root_node)
        if self.disable or len(key) == 0:
            return empty
        tokens = key.token_ids[: self._page_trunc(len(key))]
        if not tokens:
            return empty
        ns = key.namespace
        node = self.root_node
        now = time.monotonic()
        values = []
        pos = 0
        last_dev = self.root_node
        host_hit = 0
        on_host = False
        while pos < len(tokens):
            ck = self._child_key(tokens[pos:], ns, node is self.root_node)
            child = node.children.get(ck)
            if child is None:
                break
            if child.evicted and not child.backuped:
                break
            m = _match_len(child.key, tokens[pos:], self.page_size)
            if m == 0:
                break
            if m < len(child.key):
                child = self._split(child, m)
            child.last_access_time = now
            if child.evicted:
                on_host = True
                host_hit += m
            elif on_host:
                break        # device data below a host-only node cannot be used without it
            else:
                values.append(child.value)
                last_dev = child
            node = child
            pos += m
            if m < len(child.key):
                break
        out = np.concatenate(values) if values else np.empty(0, np.int32)
        return MatchResult(out, last_dev, node if host_hit else last_dev, host_hit)

    def init_load_back(self, last_host_node: TreeNode, host_hit_length: int):
        """Bring the host-only chain ending at `last_host_node` back to the device.  Returns
        `(device_indices, new_last_node)`; empty when device memory cannot be found."""
        chain = []
        n = last_host_node
        while n is not self.root_node and n.evicted:
            chain.append(n)
            n = n.parent
        chain.reverse()
        anchor = n
        if not chain:
            return np.empty(0, np.int32), last_host_node
        need = sum(len(c.key) for c in chain)
        alloc = self.token_to_kv_pool_allocator
        dp = chain[0].namespace[1] or 0
        self.inc_lock_ref(anchor)
        try:
            if alloc.available_size(dp_rank=dp) < need:
                self.evict(need - alloc.available_size(dp_rank=dp), dp_rank=dp)
            slots = alloc.alloc(need, dp_rank=dp)
        finally:
            self.dec_lock_ref(anchor)
        if slots is None:
            return np.empty(0, np.int32), anchor
        slots = np.asarray(slots, np.int32)
        host_pages = np.concatenate([c.host_value for c in chain])
        off = 0
        for c in chain:
            c.value = slots[off:off + len(c.key)].copy()
            off += len(c.key)
            self._evictable[c.namespace] += len(c.key)
        dev_pages = (slots[:: self.page_size] // self.page_size).astype(np.int64)
        t = self.controller.load([c.id for c in chain], host_pages, dev_pages)
        # one lock on the deepest node protects the whole chain until the copy is retired
        self.inc_lock_ref(chain[-1])
        self.ongoing_load[id(t)] = [chain[-1]]
        return slots, chain[-1]

    # ------------------------------------------------------------------ eviction
    def evict(self, num_tokens: int, dp_rank: int | None = None):
        if self.disable or num_tokens <= 0:
            return 0
        self.check_hicache_events()
        leaves = [n for n in self._leaves(dp_rank) if n.lock_ref == 0]
        heapq.heapify(leaves)
        freed = 0
        while freed < num_tokens and leaves:
            n = heapq.heappop(leaves)
            if n.lock_ref > 0 or n.evicted:
                continue
            if not n.backuped and self.write_policy == "write_back":
                if self.write_backup(n, blocking=True) and n.lock_ref > 0:
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

    def evict_host(self, num_pages: int) -> int:
        """Free host pages held by host-only leaves, least recently used first."""
        cands = []
        stack = [self.root_node]
        while stack:
            n = stack.pop()
            if n is not self.root_node and n.evicted and n.backuped and not n.children and n.lock_ref == 0:
                cands.append(n)
            stack.extend(n.children.values())
        heapq.heapify(cands)
        freed = 0
        while freed < num_pages and cands:
            n = heapq.heappop(cands)
            self.host_pool.free(n.host_value)
            freed += len(n.host_value)
            n.host_value = None
            p = n.parent
            del p.children[n.child_key]
            self._on_host_node_removed(n)
            if p is not self.root_node and p.evicted and p.backuped and not p.children and p.lock_ref == 0:
                heapq.heappush(cands, p)
        return freed

    def _on_host_node_removed(self, n: TreeNode):
        """A host-only node left the tree for good (hook for trees that keep more than KV on a node)."""

    def host_size_pages(self) -> int:
        return self.host_pool.num_pages - self.host_pool.available_pages()
