"""Periodic scheduler log lines and load statistics (reference
`python/sgl_jax/srt/managers/scheduler_metrics_mixin.py:31,:89`)."""

from __future__ import annotations

import logging
import time

logger = logging.getLogger(__name__)


class SchedulerMetricsMixin:
    def init_metrics(self):
        self.last_decode_stats_tic = time.perf_counter()
        self.last_prefill_stats_tic = time.perf_counter()
        self.num_generated_tokens = 0
        self.last_gen_throughput = 0.0
        self.last_input_throughput = 0.0
        self.forward_ct_decode = 0
        self.total_retracted_reqs = 0
        self.spec_num_total_accepted_tokens = 0
        self.spec_num_total_forward_ct = 0
        self.stats = {"num_prefill_batches": 0, "num_decode_batches": 0, "num_prefill_tokens": 0,
                      "num_cached_tokens": 0}

    def token_usage(self) -> tuple[int, float]:
        used = self.max_total_num_tokens - self.token_to_kv_pool_allocator.available_size() - \
            self.tree_cache.evictable_size()
        return used, used / max(self.max_total_num_tokens, 1)

    def log_prefill_stats(self, adder, can_run_list, running_bs: int):
        now = time.perf_counter()
        gap = now - self.last_prefill_stats_tic
        self.last_prefill_stats_tic = now
        self.last_input_throughput = adder.log_input_tokens / max(gap, 1e-9)
        used, usage = self.token_usage()
        self.stats["num_prefill_batches"] += 1
        self.stats["num_prefill_tokens"] += adder.log_input_tokens
        self.stats["num_cached_tokens"] += adder.log_hit_tokens
        logger.info("Prefill batch. #new-seq: %d, #new-token: %d, #cached-token: %d, token usage: %.2f, "
                    "#running-req: %d, #queue-req: %d", len(can_run_list), adder.log_input_tokens,
                    adder.log_hit_tokens, usage, running_bs, len(self.waiting_queue))

    def log_decode_stats(self, batch=None):
        now = time.perf_counter()
        gap = now - self.last_decode_stats_tic
        self.last_decode_stats_tic = now
        self.last_gen_throughput = self.num_generated_tokens / max(gap, 1e-9)
        self.num_generated_tokens = 0
        used, usage = self.token_usage()
        self.stats["num_decode_batches"] += 1
        msg = (f"Decode batch. #running-req: {len(self.running_batch.reqs) if self.running_batch else 0}, "
               f"#token: {used}, token usage: {usage:.2f}, ")
        if self.spec_algorithm is not None and self.spec_num_total_forward_ct:
            msg += f"accept len: {self.spec_num_total_accepted_tokens / self.spec_num_total_forward_ct:.2f}, "
            self.spec_num_total_accepted_tokens = self.spec_num_total_forward_ct = 0
        msg += f"gen throughput (token/s): {self.last_gen_throughput:.2f}, #queue-req: {len(self.waiting_queue)}"
        logger.info(msg)

    def get_load(self) -> dict:
        used, _ = self.token_usage()
        return {"dp_rank": 0, "num_reqs": (len(self.running_batch.reqs) if self.running_batch else 0) + len(self.waiting_queue),
                "num_waiting_reqs": len(self.waiting_queue), "num_tokens": used + sum(len(r.origin_input_ids) for r in self.waiting_queue)}
