"""Prefix cache for hybrid models whose linear-attention layers carry a recurrent state
(reference `python/sgl_jax/srt/mem_cache/unified_radix_cache.py`,
`unified_cache_components/{tree,full,recurrent}_component.py`).

A shared prefix is only usable if, besides its KV slots (the FULL component), the recurrent state
at its *end* is available (the RECURRENT component).  Nodes therefore may carry a *snapshot*: a
slot of the `RecurrentStatePool` snapshot area holding the conv window and state matrix after the
node's last token.  Matching walks the tree as usual but stops at the deepest node that has a
snapshot; the request then starts from a copy of it (copy-on-write into its own slot) and
recomputes the rest.  Snapshots are taken (a) inside every prefill step at the last multiple of the
track interval the step covers: a slot is reserved when the step is scheduled, the workers store the state there
while they run the step, and afterwards the page-aligned prefix is published and the snapshot
attached to the node ending at it (the role of the reference's `recurrent_track_interval` tracking;
the interval is a multiple of the page size); (b) at the end of a finished request when that end is
page-aligned.

Differences from the reference's component design, chosen for this runtime: snapshots may sit on
internal nodes too (the reference keeps them on leaves and drops one when its node gains a
child), and they have their own LRU over a fixed number of snapshot slots instead of riding leaf
eviction — a node can lose its snapshot and keep its KV.  State copies are not executed here:
the tree runs in the scheduler, the pools live in every tensor rank, so copies are queued
(`take_recurrent_copies`) and travel with the next batch to all ranks, in order.

The snapshot logic is a mixin over the tree that stores the KV (`UnifiedRadixCache`: the plain radix tree;
`UnifiedHiRadixCache`: the tree with a host-memory tier, the reference's HiCache hooks `write_backup` :835,
`evict_host` :1022, `init_load_back` :1061).  With the host tier a node whose KV was demoted to the host keeps its
snapshot (snapshots are small and have their own LRU), so a later request can match through host-only nodes up to the
deepest checkpoint, have the KV of that chain loaded back and start from the checkpoint; if the load-back finds no
device memory the request falls back to the deepest checkpoint whose KV is still on the device.
"""

from __future__ import annotations

from collections import OrderedDict
from enum import IntEnum

import numpy as np

from .base_prefix_cache import MatchResult
from .hiradix_cache import HiRadixCache
from .radix_cache import RadixCache, RadixKey, TreeNode


class ComponentType(IntEnum):
    FULL = 0
    RECURRENT = 1


class _RecurrentSnapshots:
    """Checkpoints of the recurrent state on tree nodes; mixed into a radix tree class (see the module docstring)."""

    def _init_snapshots(self, page_size: int, num_request_slots: int, num_snapshot_slots: int,
                        track_interval: int | None, commit_on_finish: bool, recurrent: bool = True):
        # `--enable-unified-radix-tree` selects this tree for models without linear-attention layers too: with the
        # FULL component alone every hook below hands over to the tree underneath
        self.components = (ComponentType.FULL, ComponentType.RECURRENT) if recurrent else (ComponentType.FULL,)
        self.recurrent = recurrent
        # checkpoint the final state of a finished request from its own slot: only sound when no overlapped extra
        # decode step can have advanced that slot past the request's last cached token
        self.commit_on_finish = commit_on_finish
        # prefill checkpoints sit on multiples of this many tokens (a multiple of the page size)
        self.track_interval = int(track_interval or page_size)
        if self.track_interval <= 0 or self.track_interval % page_size:
            raise ValueError(f"recurrent_track_interval ({self.track_interval}) must be a positive multiple of the "
                             f"page size ({page_size})")
        self.snapshot_base = num_request_slots + 1          # request row r owns state slot r + 1
        self.num_snapshot_slots = num_snapshot_slots

    # ---------------------------------------------------------------- state
    def reset(self):
        super().reset()
        self._snap: dict[int, int] = {}                     # node id -> snapshot slot
        self._nodes: dict[int, TreeNode] = {}               # node id -> node, for snapshot holders
        self._lru: OrderedDict[int, None] = OrderedDict()   # node ids, least recently used first
        self._free_snap = list(range(self.snapshot_base, self.snapshot_base + self.num_snapshot_slots))
        self._copies: list[tuple[int, int]] = []
        # request id -> [aligned length, tokens of the extend before it, snapshot slot, sent to the workers]
        self._pending_track: dict[str, list] = {}
        self._raw_match = False
        # host-tier matches: id of the host-only checkpoint node -> the device checkpoint node the match fell back to
        self._load_stop: dict[int, TreeNode] = {}

    def supports_recurrent(self) -> bool:
        return self.recurrent

    def take_recurrent_copies(self) -> list[tuple[int, int]]:
        """(src slot, dst slot) state copies to run, in order, before the next forward."""
        c, self._copies = self._copies, []
        return c

    def queue_copy(self, src: int, dst: int):
        self._copies.append((int(src), int(dst)))

    def recurrent_evictable_size(self) -> int:
        return sum(1 for i in self._snap if self._nodes[i].lock_ref == 0)

    def snapshot_slots_in_use(self) -> int:
        return len(self._snap)

    def assert_recurrent_slot_ledger(self):
        used = sorted(list(self._snap.values()) + [t[2] for t in self._pending_track.values()])
        assert len(set(used)) == len(used), "a snapshot slot is owned twice"
        assert sorted(used + self._free_snap) == list(range(self.snapshot_base,
                                                            self.snapshot_base + self.num_snapshot_slots)), \
            "snapshot slots leaked"
        return len(used)

    # ---------------------------------------------------------------- match
    def match_prefix(self, key: RadixKey, req=None, **kw) -> MatchResult:
        res = super().match_prefix(key)
        if self._raw_match or not self.recurrent:
            return res                                    # re-pointing a running request at its own prefix
        root = self.root_node
        empty = MatchResult(np.empty(0, np.int32), root, root)
        deepest = res.last_host_node if res.host_hit_length else res.last_device_node
        if req is not None:
            req.recurrent_cow_src = None
        if self.disable or deepest is None or deepest is root:
            return empty
        path = []
        n = deepest
        while n is not root:
            path.append(n)
            n = n.parent
        path.reverse()
        # deepest node with the recurrent state at its end: on the whole matched path, and on its device part
        dev_total = len(res.device_indices)
        cum = 0
        on_dev = on_any = None
        for n in path:
            cum += len(n.key)
            if n.id in self._snap:
                on_any = (n, cum)
                if cum <= dev_total and not n.evicted:
                    on_dev = (n, cum)
        if on_any is None:
            return empty
        self._lru.move_to_end(on_any[0].id)
        if on_dev is not None:
            self._lru.move_to_end(on_dev[0].id)
        if on_any is on_dev or on_any[1] <= dev_total:
            node, total = on_any
            if req is not None:
                req.recurrent_cow_src = self._snap[node.id]
            return MatchResult(res.device_indices[:total], node, node)
        # the deepest checkpoint sits on a node whose KV is on the host tier: report the device part up to the
        # deepest device checkpoint and the rest as a host hit; `init_load_back` completes it
        dev_node, dev_len = on_dev if on_dev is not None else (root, 0)
        host_node, host_end = on_any
        self._load_stop[host_node.id] = dev_node
        if req is not None:
            req.recurrent_cow_src = self._snap[(dev_node if on_dev is not None else host_node).id]
        return MatchResult(res.device_indices[:dev_len], dev_node, host_node, host_end - dev_len)

    # ---------------------------------------------------------------- request hooks
    def cache_finished_req(self, req, is_insert: bool = True, **kw):
        if not self.recurrent:
            return super().cache_finished_req(req, is_insert, **kw)
        track = self._pending_track.pop(req.rid, None)       # finished / aborted before its prefill was published
        if track is not None:
            self._free_snap.append(track[2])
        kv_len = req.committed_kv_len()
        tokens = (req.origin_input_ids + req.output_ids)[:kv_len]
        row = req.req_pool_idx
        super().cache_finished_req(req, is_insert, **kw)
        if self.disable or not self.commit_on_finish or not is_insert or kv_len == 0 or kv_len % self.page_size:
            return          # the state belongs to position kv_len; only a node ending there can own it
        dp = getattr(req, "dp_rank", 0) or 0
        values, node = self._match(tokens, RadixKey(tokens, req.extra_key, dp).namespace)
        if node is self.root_node or sum(len(v) for v in values) != kv_len or node.id in self._snap:
            return
        slot = self._alloc_snapshot()
        if slot is None:
            return
        self._snap[node.id] = slot
        self._nodes[node.id] = node
        self._lru[node.id] = None
        self.queue_copy(row + 1, slot)

    def cache_unfinished_req(self, req, chunked: bool = False, **kw):
        """After a prefill step.  Without a checkpoint inside the step the state exists only in the request's own
        slot and nothing is published.  With one (`on_extend_scheduled`), the page-aligned prefix goes into the
        tree like in a plain radix cache and the checkpoint is attached to the node that ends at it."""
        if not self.recurrent:
            return super().cache_unfinished_req(req, chunked, **kw)
        track = self._pending_track.pop(req.rid, None)
        if self.disable or track is None or not track[3]:
            if track is not None:
                self._free_snap.append(track[2])
            kv_len = len(req.fill_ids)
            req.prefix_indices = self.req_to_token_pool.read(req.req_pool_idx, kv_len).copy()
            return
        aligned, _, slot, _ = track
        self._raw_match = True
        try:
            super().cache_unfinished_req(req, chunked, **kw)
        finally:
            self._raw_match = False
        dp = getattr(req, "dp_rank", 0) or 0
        tokens = req.fill_ids[:aligned]
        values, node = self._match(tokens, RadixKey(tokens, req.extra_key, dp).namespace)
        if node is self.root_node or sum(len(v) for v in values) != aligned or node.id in self._snap:
            self._free_snap.append(slot)
            return
        self._snap[node.id] = slot
        self._nodes[node.id] = node
        self._lru[node.id] = None

    def on_extend_scheduled(self, req, prefix_len: int, seq_len: int):
        """A prefill step covering tokens `[prefix_len, seq_len)` is about to run: if a page boundary falls inside
        it, reserve a snapshot slot and ask the workers to store the state at the last such boundary."""
        if self.disable or not self.recurrent:
            return
        old = self._pending_track.pop(req.rid, None)
        if old is not None:
            self._free_snap.append(old[2])
        aligned = seq_len // self.track_interval * self.track_interval
        if aligned <= prefix_len or aligned <= 0:
            return
        slot = self._alloc_snapshot()
        if slot is None:
            return
        self._pending_track[req.rid] = [aligned, aligned - prefix_len, slot, False]

    def take_recurrent_tracks(self, reqs) -> list[tuple[int, int, int]]:
        """(index in the batch, tokens of the extend before the checkpoint, snapshot slot) per request."""
        out = []
        for i, r in enumerate(reqs):
            t = self._pending_track.get(r.rid)
            if t is not None:
                t[3] = True
                out.append((i, t[1], t[2]))
        return out

    def on_request_scheduled(self, req):
        """First prefill of a request that matched a snapshot: clone it into the request's slot.  The request's last
        node decides which one: after a load-back from the host tier it is the deeper checkpoint."""
        src = getattr(req, "recurrent_cow_src", None)
        if src is not None and len(req.prefix_indices) > 0:
            node = getattr(req, "last_node", None)
            if node is not None and getattr(node, "id", None) in self._snap:
                src = self._snap[node.id]
            self.queue_copy(src, req.req_pool_idx + 1)
        req.recurrent_cow_src = None

    # ---------------------------------------------------------------- snapshots
    def _alloc_snapshot(self) -> int | None:
        if self._free_snap:
            return self._free_snap.pop()
        for nid in self._lru:                    # least recently used, not pinned by a running request
            if self._nodes[nid].lock_ref == 0:
                return self._release_snapshot(nid, reuse=True)
        return None

    def _release_snapshot(self, nid: int, reuse: bool = False):
        slot = self._snap.pop(nid)
        self._nodes.pop(nid, None)
        self._lru.pop(nid, None)
        if reuse:
            return slot
        self._free_snap.append(slot)
        return None

    def _drop(self, n: TreeNode):
        # a node that stays in the tree as a host-only node keeps its checkpoint
        if n.id in self._snap and not n.backuped:
            self._release_snapshot(n.id)
        super()._drop(n)

    def _on_host_node_removed(self, n: TreeNode):
        if n.id in self._snap:
            self._release_snapshot(n.id)
        self._load_stop.pop(n.id, None)


class UnifiedRadixCache(_RecurrentSnapshots, RadixCache):
    def __init__(self, req_to_token_pool, token_to_kv_pool_allocator, page_size: int = 1, disable: bool = False,
                 num_request_slots: int = 0, num_snapshot_slots: int = 0, enable_kv_cache_events: bool = False,
                 track_interval: int | None = None, commit_on_finish: bool = True, recurrent: bool = True):
        self._init_snapshots(page_size, num_request_slots, num_snapshot_slots, track_interval, commit_on_finish,
                             recurrent)
        RadixCache.__init__(self, req_to_token_pool, token_to_kv_pool_allocator, page_size, disable,
                            enable_kv_cache_events)


class UnifiedHiRadixCache(_RecurrentSnapshots, HiRadixCache):
    """FULL + RECURRENT components over the tree with a host-memory KV tier."""

    def __init__(self, req_to_token_pool, token_to_kv_pool_allocator, page_size: int, device_pool,
                 num_request_slots: int = 0, num_snapshot_slots: int = 0, track_interval: int | None = None,
                 commit_on_finish: bool = True, hicache_ratio: float = 2.0, write_policy: str = "write_through",
                 write_through_threshold: int = 1, host_pages: int | None = None, disable: bool = False,
                 enable_kv_cache_events: bool = False, recurrent: bool = True):
        self._init_snapshots(page_size, num_request_slots, num_snapshot_slots, track_interval, commit_on_finish,
                             recurrent)
        HiRadixCache.__init__(self, req_to_token_pool, token_to_kv_pool_allocator, page_size, device_pool,
                              hicache_ratio, write_policy, write_through_threshold, host_pages, disable=disable,
                              enable_kv_cache_events=enable_kv_cache_events)

    def init_load_back(self, last_host_node: TreeNode, host_hit_length: int):
        """Host-tier trees only.  The host hit of a checkpoint match spans the device-resident nodes between the device
        checkpoint and the host-only chain, then the chain itself: return the slots of both, in order."""
        root = self.root_node
        stop = self._load_stop.pop(last_host_node.id, root)
        n = last_host_node
        while n is not root and n.evicted:
            n = n.parent
        middle = []
        while n is not root and n is not stop:
            middle.append(n)
            n = n.parent
        if n is not stop:
            return np.empty(0, np.int32), stop            # the tree changed under the match: keep the device part
        slots, new_last = super().init_load_back(last_host_node, host_hit_length)
        if not len(slots):
            return slots, stop
        middle.reverse()
        return np.concatenate([m.value for m in middle] + [slots]).astype(np.int32), new_last
