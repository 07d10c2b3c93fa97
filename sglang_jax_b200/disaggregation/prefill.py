"""Prefill side of PD disaggregation (reference
`python/sgl_jax/srt/disaggregation/prefill.py`: `SchedulerDisaggregationPrefillMixin` :227).

A request with a `bootstrap_room` runs its prefill here and produces exactly one token.  When
it finishes, its KV pages are not released: they are published under the room id, the decode
engine pulls them, and only the decode engine's acknowledgement (or the timeout reaper) lets
the request go through the usual finish path that hands the pages to the prefix cache."""

from __future__ import annotations

import logging
import time
import uuid

import numpy as np

from . import req_time_stats
from .base.kv_manager import KVPoll
from .common import metrics

logger = logging.getLogger(__name__)


class SchedulerDisaggregationPrefillMixin:
    def init_disaggregation_prefill(self):
        from .runtime import build_kv_manager
        sa = self.server_args
        self.disagg_engine_id = getattr(sa, "disaggregation_engine_id", None) or f"prefill-{uuid.uuid4().hex[:8]}"
        self.disagg_kv_manager, self.disagg_heartbeat = build_kv_manager(self, "prefill", self.disagg_engine_id)
        self.disagg_prefill_inflight: list = []
        self.disagg_sent = 0
        self.disagg_failed = 0

    # called at request intake
    def disagg_prefill_admit(self, req) -> None:
        if req.bootstrap_room is None:
            return
        req.sampling_params.max_new_tokens = 1      # the decode engine generates the rest
        req.sampling_params.ignore_eos = True
        req.stream = False

    # called by `_finish_req` instead of releasing the KV; returns True when it took the request over
    def disagg_prefill_hold(self, req) -> bool:
        if req.bootstrap_room is None or getattr(req, "disagg_done", False) or req.req_pool_idx is None:
            return False
        from ..managers.schedule_batch import FINISH_ABORT
        if isinstance(req.finished_reason, FINISH_ABORT) or not req.output_ids:
            return False
        P = self.page_size
        # only the prompt's KV is handed over (an overlapped decode step may already have
        # appended one more slot, which the decode engine recomputes itself)
        kv_len = min(req.kv_committed_len, len(req.origin_input_ids))
        slots = self.req_to_token_pool.read(req.req_pool_idx, kv_len)
        pages = (slots[::P] // P).astype(np.int64)
        req_time_stats.mark(self, req, "forward_done")
        try:
            sender = self.disagg_kv_manager.create_sender(req.rid)
            sender.init(pages, str(req.bootstrap_room), int(req.output_ids[0]),
                        {"prompt_len": len(req.origin_input_ids), "kv_len": int(kv_len), "rid": req.rid})
            sender.send()
        except Exception as e:  # noqa: BLE001
            logger.error("could not publish KV of %s: %s", req.rid, e)
            return False
        req.disagg_sender = sender
        req.disagg_sent_time = time.perf_counter()
        req_time_stats.mark(self, req, "transfer_start")
        self.disagg_prefill_inflight.append(req)
        metrics.set_queue_depth("prefill_inflight", len(self.disagg_prefill_inflight))
        return True

    # called every scheduler iteration
    def process_disagg_prefill_inflight(self) -> int:
        if not self.disagg_prefill_inflight:
            return 0
        keep, done = [], 0
        for req in self.disagg_prefill_inflight:
            st = req.disagg_sender.poll()
            if not st.terminal:
                keep.append(req)
                continue
            if st == KVPoll.SUCCESS:
                self.disagg_sent += 1
            else:
                self.disagg_failed += 1
                logger.warning("KV transfer of %s failed: %s", req.rid, req.disagg_sender.state.failure)
            req.disagg_sender.clear()
            req.disagg_done = True
            req_time_stats.mark(self, req, "transfer_done", final=True)
            # a failed hand-over leaves nothing worth caching under this engine's name either way;
            # the pages are valid KV of the prompt, so they can serve later prefixes
            self._finish_req(req)
            done += 1
        self.disagg_prefill_inflight = keep
        metrics.set_queue_depth("prefill_inflight", len(keep))
        return done
