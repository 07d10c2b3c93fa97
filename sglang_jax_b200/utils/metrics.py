"""Prometheus metrics (reference: `--enable-metrics` mounts `/metrics` with the multiprocess
collector, `python/sgl_jax/srt/utils/common_utils.py:187-216`; histogram bucket flags
`--bucket-time-to-first-token / -inter-token-latency / -e2e-request-latency`)."""

from __future__ import annotations

import time


class TokenizerMetricsCollector:
    def __init__(self, server_args):
        from prometheus_client import Counter, Histogram
        labels = {"model_name": server_args.served_model_name}
        self.labels = labels
        ln = list(labels)
        ttft = server_args.bucket_time_to_first_token or [0.1, 0.25, 0.5, 0.75, 1, 2, 5, 10, 20, 40, 60, 80, 120, 160]
        itl = server_args.bucket_inter_token_latency or [0.002, 0.004, 0.006, 0.008, 0.01, 0.015, 0.02, 0.025, 0.03,
                                                         0.04, 0.05, 0.075, 0.1, 0.15, 0.2, 0.3, 0.4, 0.5, 1, 2]
        e2e = server_args.bucket_e2e_request_latency or [0.1, 0.25, 0.5, 1, 2, 5, 10, 20, 40, 60, 80, 100, 150, 200]
        self.prompt_tokens_total = Counter("sglang:prompt_tokens_total", "Number of prefill tokens processed.", ln)
        self.generation_tokens_total = Counter("sglang:generation_tokens_total", "Number of generation tokens processed.", ln)
        self.cached_tokens_total = Counter("sglang:cached_tokens_total", "Number of cached prompt tokens.", ln)
        self.num_requests_total = Counter("sglang:num_requests_total", "Number of requests processed.", ln)
        self.num_aborted_requests_total = Counter("sglang:num_aborted_requests_total", "Number of requests aborted.", ln)
        self.histogram_time_to_first_token = Histogram("sglang:time_to_first_token_seconds",
                                                       "Histogram of time to first token in seconds.", ln, buckets=ttft)
        self.histogram_inter_token_latency = Histogram("sglang:inter_token_latency_seconds",
                                                       "Histogram of inter-token latency in seconds.", ln, buckets=itl)
        self.histogram_e2e_request_latency = Histogram("sglang:e2e_request_latency_seconds",
                                                       "Histogram of End-to-end request latency in seconds", ln, buckets=e2e)
        self._last = {}

    def observe(self, state, meta: dict, finished: bool):
        rid = meta["id"]
        now = time.time()
        n = meta.get("completion_tokens", 0)
        last_t, last_n = self._last.get(rid, (None, 0))
        if last_t is None:
            self.histogram_time_to_first_token.labels(**self.labels).observe(now - state.created_time)
        elif n > last_n:
            self.histogram_inter_token_latency.labels(**self.labels).observe((now - last_t) / (n - last_n))
        self._last[rid] = (now, n)
        if finished:
            self._last.pop(rid, None)
            self.prompt_tokens_total.labels(**self.labels).inc(meta.get("prompt_tokens", 0))
            self.generation_tokens_total.labels(**self.labels).inc(n)
            self.cached_tokens_total.labels(**self.labels).inc(meta.get("cached_tokens", 0))
            self.num_requests_total.labels(**self.labels).inc(1)
            fr = meta.get("finish_reason") or {}
            if fr.get("type") == "abort":
                self.num_aborted_requests_total.labels(**self.labels).inc(1)
            self.histogram_e2e_request_latency.labels(**self.labels).observe(now - state.created_time)


class SchedulerMetricsCollector:
    def __init__(self, server_args):
        from prometheus_client import Gauge
        self.labels = {"model_name": server_args.served_model_name}
        ln = list(self.labels)
        mk = lambda n, d: Gauge(n, d, ln, multiprocess_mode="mostrecent")  # noqa: E731
        self.num_running_reqs = mk("sglang:num_running_reqs", "The number of running requests.")
        self.num_queue_reqs = mk("sglang:num_queue_reqs", "The number of requests in the waiting queue.")
        self.token_usage = mk("sglang:token_usage", "The token usage.")
        self.gen_throughput = mk("sglang:gen_throughput", "The generation throughput (token/s).")
        self.cache_hit_rate = mk("sglang:cache_hit_rate", "The prefix cache hit rate.")
        self.spec_accept_length = mk("sglang:spec_accept_length", "The average acceptance length of speculative decoding.")

    def log(self, running, queued, usage, throughput, hit_rate=0.0, accept_len=0.0):
        for g, v in ((self.num_running_reqs, running), (self.num_queue_reqs, queued), (self.token_usage, usage),
                     (self.gen_throughput, throughput), (self.cache_hit_rate, hit_rate),
                     (self.spec_accept_length, accept_len)):
            g.labels(**self.labels).set(v)
