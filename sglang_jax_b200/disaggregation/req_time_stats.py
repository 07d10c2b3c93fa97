"""Per-request timestamps of the PD pipeline (reference
`python/sgl_jax/srt/disaggregation/req_time_stats.py`)."""

from __future__ import annotations

import dataclasses
import time


@dataclasses.dataclass
class ReqTimeStats:
    created: float = dataclasses.field(default_factory=time.perf_counter)
    prealloc_done: float | None = None
    transfer_start: float | None = None
    transfer_done: float | None = None
    first_decode_step: float | None = None
    finished: float | None = None

    def mark(self, name: str):
        setattr(self, name, time.perf_counter())

    def durations(self) -> dict:
        def d(a, b):
            return None if a is None or b is None else b - a
        return {"queue_s": d(self.created, self.prealloc_done), "transfer_s": d(self.transfer_start, self.transfer_done),
                "wait_decode_s": d(self.transfer_done, self.first_decode_step),
                "total_s": d(self.created, self.finished)}
