"""Decode side of PD disaggregation (reference `python/sgl_jax/srt/disaggregation/decode.py`:
`DecodePreallocQueue` :94, `DecodeTransferQueue` :138, mixin :195, event loop :204-246).

A request with a `bootstrap_room` never prefills here.  It waits in the *prealloc queue* until
the KV pool can hold its prompt while keeping `num_reserved_decode_tokens` free per running
request; then a row and pages are reserved and a receiver starts pulling.  The *transfer
queue* polls the receivers; a finished pull turns the request into an ordinary decoding
request whose first token came from the prefill engine."""

from __future__ import annotations

import logging
import time

import numpy as np

from . import req_time_stats
from .base.kv_manager import KVPoll
from .common import metrics

logger = logging.getLogger(__name__)


class DecodePreallocQueue:
    def __init__(self, scheduler):
        self.s = scheduler
        self.queue: list = []

    def add(self, req):
        req.disagg_enqueue_time = time.perf_counter()
        req_time_stats.mark(self.s, req, "created")
        self.queue.append(req)
        metrics.set_queue_depth("decode_prealloc", len(self.queue))

    def _capacity_ok(self, need_tokens: int) -> bool:
        s = self.s
        sa = s.server_args
        reserve = sa.disaggregation_num_reserved_decode_tokens * (len(s.running_batch.reqs) + len(s.disagg_transfer_queue.queue) + 1)
        avail = s.token_to_kv_pool_allocator.available_size() + s.tree_cache.evictable_size()
        return avail - need_tokens >= min(reserve, s.max_total_num_tokens // 2)

    def pop_preallocated(self) -> list:
        """Reserve a row + pages for as many queued requests as capacity allows and start
        their pulls; returns the requests that moved on."""
        s = self.s
        out, keep = [], []
        max_inflight = s.server_args.disaggregation_max_inflight_transfers
        for req in self.queue:
            if req.finished():                      # aborted while waiting
                s.stream_output([req], False)
                continue
            n = len(req.origin_input_ids)
            P = s.page_size
            need = (n + P - 1) // P * P
            if (len(s.disagg_transfer_queue.queue) + len(out) >= max_inflight or keep
                    or s.req_to_token_pool.available_size() <= 0 or not self._capacity_ok(need)
                    or len(s.running_batch.reqs) + len(s.disagg_transfer_queue.queue) + len(out) >= s.max_running_requests):
                keep.append(req)
                continue
            addr = s.disagg_resolve_prefill(req)
            if addr is None:
                if time.perf_counter() - req.disagg_enqueue_time > s.server_args.disaggregation_bootstrap_timeout_seconds:
                    s.disagg_fail(req, "no live prefill engine is registered for this request")
                else:
                    keep.append(req)
                continue
            alloc = s.token_to_kv_pool_allocator
            if alloc.available_size() < need:
                s.tree_cache.evict(need - alloc.available_size())
            slots = alloc.alloc_extend(np.zeros(1, np.int32), np.asarray([n], np.int32), np.full(1, -1, np.int32), n) \
                if P > 1 else alloc.alloc(n)
            if slots is None:
                keep.append(req)
                continue
            row = s.req_to_token_pool.alloc(1)
            if row is None:
                alloc.free(slots)
                keep.append(req)
                continue
            req.req_pool_idx = int(row[0]) if hasattr(row, "__len__") else int(row)
            slots = np.asarray(slots, np.int32)
            s.req_to_token_pool.write(req.req_pool_idx, 0, slots)
            req.kv_allocated_len = n
            req.prefix_indices = np.empty(0, np.int32)
            req.last_node = s.tree_cache.root_node if hasattr(s.tree_cache, "root_node") else None
            req.last_matched_prefix_len = 0
            req.fill_ids = list(req.origin_input_ids)
            pages = (slots[::P] // P).astype(np.int64)
            recv = s.disagg_kv_manager.create_receiver(req.rid)
            recv.init(pages, str(req.bootstrap_room), addr)
            req.disagg_receiver = recv
            req_time_stats.mark(s, req, "prealloc_done")
            out.append(req)
        self.queue = keep
        metrics.set_queue_depth("decode_prealloc", len(keep))
        return out


class DecodeTransferQueue:
    def __init__(self, scheduler):
        self.s = scheduler
        self.queue: list = []

    def extend(self, reqs):
        self.queue.extend(reqs)
        metrics.set_queue_depth("decode_transfer", len(self.queue))

    def pop_transferred(self) -> list:
        s = self.s
        done, keep = [], []
        for req in self.queue:
            st = req.disagg_receiver.poll()
            if st == KVPoll.SUCCESS:
                meta = req.disagg_receiver.meta or {}
                req.disagg_receiver.clear()
                n = len(req.origin_input_ids)
                if int(meta.get("kv_len", n)) != n:
                    s.disagg_fail(req, f"prefill engine cached {meta.get('kv_len')} tokens for a prompt of {n}")
                    continue
                req.output_ids = [int(meta["first_token"])]
                req.kv_committed_len = n
                req.first_token_time = time.perf_counter()
                req_time_stats.mark(s, req, "transfer_done")
                done.append(req)
            elif st == KVPoll.FAILED:
                reason = req.disagg_receiver.state.failure
                req.disagg_receiver.clear()
                s.disagg_fail(req, f"KV transfer failed: {reason}")
            elif req.to_abort:
                req.disagg_receiver.abort()
                req.disagg_receiver.clear()
                s.disagg_fail(req, req.to_abort_message or "Aborted")
            else:
                keep.append(req)
        self.queue = keep
        metrics.set_queue_depth("decode_transfer", len(keep))
        return done


class SchedulerDisaggregationDecodeMixin:
    def init_disaggregation_decode(self):
        from .bootstrap import BootstrapClient, PrefillInfoCache
        from .runtime import build_kv_manager, kv_layout_of
        sa = self.server_args
        self.disagg_engine_id = getattr(sa, "disaggregation_engine_id", None) or "decode"
        self.disagg_kv_manager, _ = build_kv_manager(self, "decode", self.disagg_engine_id)
        self.disagg_prealloc_queue = DecodePreallocQueue(self)
        self.disagg_transfer_queue = DecodeTransferQueue(self)
        self.disagg_prefill_cache = PrefillInfoCache(
            BootstrapClient(sa.disaggregation_bootstrap_url, sa.disaggregation_shared_secret,
                            sa.disaggregation_bootstrap_timeout_seconds), kv_layout_of(self))
        self.disagg_received = 0
        self.disagg_failed = 0
        # `--disaggregation-decode-watchdog-seconds`: complain when the loop has not turned for that long although
        # requests wait in the prealloc / transfer queues or decode (reference `runtime.py:136`)
        from .decode_watchdog import EventLoopWatchdog
        self.disagg_decode_watchdog = EventLoopWatchdog(
            float(getattr(sa, "disaggregation_decode_watchdog_seconds", 0) or 0),
            has_work=lambda: bool(self.disagg_prealloc_queue.queue or self.disagg_transfer_queue.queue
                                  or not self.running_batch.is_empty()),
            on_stall=lambda idle: logger.error(
                "PD decode loop has not turned for %.1fs: prealloc=%d transfer=%d running=%d", idle,
                len(self.disagg_prealloc_queue.queue), len(self.disagg_transfer_queue.queue),
                len(self.running_batch.reqs))).start()

    def disagg_decode_admit(self, req) -> bool:
        """Route a PD request into the prealloc queue; False = treat as an ordinary request."""
        if req.bootstrap_room is None:
            return False
        self.disagg_prealloc_queue.add(req)
        return True

    def disagg_resolve_prefill(self, req) -> str | None:
        if req.bootstrap_host and req.bootstrap_port:
            return f"{req.bootstrap_host}:{req.bootstrap_port}"
        e = self.disagg_prefill_cache.lookup(req.bootstrap_host, 0, room=int(req.bootstrap_room))
        return e["transfer_addr"] if e else None

    def disagg_fail(self, req, message: str):
        from ..managers.schedule_batch import FINISH_ABORT
        self.disagg_failed += 1
        if req.req_pool_idx is not None:
            slots = self.req_to_token_pool.read(req.req_pool_idx, req.kv_allocated_len).copy()
            self.token_to_kv_pool_allocator.free(slots)
            self.req_to_token_pool.free(req.req_pool_idx)
            req.req_pool_idx = None
        req.finished_reason = FINISH_ABORT(message, 502, "KVTransferError")
        self.stream_output([req], False)

    def process_disagg_decode_queues(self) -> int:
        """One turn of the decode-side pipeline: prealloc -> transfer -> running batch."""
        self.disagg_decode_watchdog.beat()
        moved = self.disagg_prealloc_queue.pop_preallocated()
        if moved:
            self.disagg_transfer_queue.extend(moved)
        ready = self.disagg_transfer_queue.pop_transferred()
        if not ready:
            return 0
        from ..managers.schedule_batch import ScheduleBatch
        alive = []
        for req in ready:
            self.disagg_received += 1
            if req.grammar is not None:
                req.grammar.accept_token(req.output_ids[0])
            req.check_finished()
            if req.finished():
                self._finish_req(req)
            else:
                alive.append(req)
        self.stream_output(ready, False)
        if alive:
            nb = ScheduleBatch.init_new(alive, self.req_to_token_pool, self.token_to_kv_pool_allocator, self.tree_cache,
                                        self.vocab_size, self.enable_overlap, self.page_size, self.spec_algorithm)
            nb.prepare_for_transferred_decode()
            if self.running_batch.is_empty():
                self.running_batch = nb
            else:
                self.running_batch.merge_batch(nb)
        return len(ready)
