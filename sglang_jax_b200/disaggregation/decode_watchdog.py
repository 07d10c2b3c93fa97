"""Detects a decode event loop that stopped turning (reference
`python/sgl_jax/srt/disaggregation/decode_watchdog.py:34`): the loop calls `beat()` every
iteration; when no beat arrives for `timeout` seconds while work is pending, `on_stall` runs
(by default it logs the queues and raises in the watchdog thread's owner via the callback)."""

from __future__ import annotations

import logging
import threading
import time
from typing import Callable

logger = logging.getLogger(__name__)


class EventLoopWatchdog:
    def __init__(self, timeout: float, has_work: Callable[[], bool], on_stall: Callable[[float], None] | None = None,
                 poll: float | None = None):
        self.timeout = timeout
        self.has_work = has_work
        self.on_stall = on_stall or (lambda idle: logger.error("decode event loop stalled for %.1fs", idle))
        self._last = time.monotonic()
        self._stop = threading.Event()
        self.stalls = 0
        self._poll = poll if poll is not None else max(min(timeout / 4, 1.0), 0.01)
        self._thread = threading.Thread(target=self._run, daemon=True, name="pd-decode-watchdog")

    def start(self):
        if self.timeout and self.timeout > 0:
            self._thread.start()
        return self

    def beat(self):
        self._last = time.monotonic()

    def _run(self):
        while not self._stop.wait(self._poll):
            idle = time.monotonic() - self._last
            if idle > self.timeout and self.has_work():
                self.stalls += 1
                try:
                    self.on_stall(idle)
                finally:
                    self._last = time.monotonic()

    def stop(self):
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=2)
