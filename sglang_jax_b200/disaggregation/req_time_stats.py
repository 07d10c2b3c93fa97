"""Per-request timestamps of the PD pipeline (reference
`python/sgl_jax/srt/disaggregation/req_time_stats.py`, the `_pd_mark_time` calls of `prefill.py` / `decode.py`).
Active with `--enable-request-time-stats-logging`: the schedulers mark the stages a request passes and log one line
per request when it leaves the engine."""

from __future__ import annotations

import logging
import time

logger = logging.getLogger(__name__)

# stage marks in pipeline order, per role
STAGES = {
    "prefill": ("created", "forward_done", "transfer_start", "transfer_done"),
    "decode": ("created", "prealloc_done", "transfer_done", "first_decode_step", "finished"),
}


class ReqTimeStats:
    def __init__(self, role: str = "decode"):
        self.role = role
        self.marks: dict[str, float] = {"created": time.perf_counter()}

    def mark(self, name: str):
        self.marks.setdefault(name, time.perf_counter())

    def durations(self) -> dict:
        """Seconds spent between consecutive marked stages (stages that were never reached are left out)."""
        out, prev = {}, None
        for name in STAGES.get(self.role, ()):
            t = self.marks.get(name)
            if t is None:
                continue
            if prev is not None:
                out[f"{prev[0]}->{name}"] = t - prev[1]
            prev = (name, t)
        if prev is not None:
            out["total_s"] = prev[1] - self.marks["created"]
        return out


def mark(scheduler, req, name: str, final: bool = False):
    """Record stage `name` on `req` when the scheduler has time-stats logging on; `final` also logs the line."""
    if not getattr(scheduler.server_args, "enable_request_time_stats_logging", False):
        return
    ts = getattr(req, "pd_time_stats", None)
    if ts is None:
        ts = req.pd_time_stats = ReqTimeStats(scheduler.server_args.disaggregation_mode or "decode")
    ts.mark(name)
    if final:
        logger.info("PD time stats rid=%s role=%s %s", req.rid, ts.role,
                    " ".join(f"{k}={v * 1e3:.1f}ms" for k, v in ts.durations().items()))
