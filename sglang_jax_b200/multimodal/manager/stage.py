"""One pipeline stage: devices, an input queue, a scheduler thread that batches requests and
runs the stage's executor, and an output queue (reference `multimodal/manager/stage.py`)."""

from __future__ import annotations

import logging
import queue
import threading
import time

from ..configs.stage_config import StageConfig
from .io_struct import MMReq

logger = logging.getLogger(__name__)


class Stage:
    def __init__(self, config: StageConfig, devices: list[str], scheduler):
        self.config = config
        self.devices = devices
        self.scheduler = scheduler
        self.in_queue: "queue.Queue[MMReq | None]" = queue.Queue()
        self.out_queue: "queue.Queue[MMReq] | None" = None        # wired by the global scheduler
        self.aborted: set[str] = set()
        self._lock = threading.Lock()
        self._thread = threading.Thread(target=self._run, daemon=True, name=f"mm-stage-{config.stage_id}")
        self.processed = 0

    def start(self):
        self._thread.start()

    def stop(self):
        self.in_queue.put(None)
        self._thread.join(timeout=10)
        if hasattr(self.scheduler, "shutdown"):
            self.scheduler.shutdown()

    def abort(self, rid: str):
        with self._lock:
            self.aborted.add(rid)
        self.scheduler.abort(rid)

    def _take_batch(self) -> list[MMReq] | None:
        first = self.in_queue.get()
        if first is None:
            return None
        batch = [first]
        while len(batch) < self.config.max_batch_size:
            try:
                nxt = self.in_queue.get_nowait()
            except queue.Empty:
                break
            if nxt is None:
                self.in_queue.put(None)
                break
            batch.append(nxt)
        return batch

    def _run(self):
        while True:
            batch = self._take_batch()
            if batch is None:
                return
            with self._lock:
                live = [r for r in batch if r.rid not in self.aborted and not r.aborted]
                for r in batch:
                    if r.rid in self.aborted:
                        r.aborted = True
                        self.aborted.discard(r.rid)
            t0 = time.perf_counter()
            if live:
                try:
                    self.scheduler.run_batch(live)
                except Exception as e:  # noqa: BLE001
                    logger.exception("stage %d failed", self.config.stage_id)
                    for r in live:
                        r.error = f"stage {self.config.stage_id} ({self.config.scheduler}): {e}"
            dt = time.perf_counter() - t0
            for r in batch:
                r.stage_times[self.config.stage_id] = dt
                self.processed += 1
                self.out_queue.put(r)
