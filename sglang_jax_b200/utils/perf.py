"""Kernel timing helper (reference `python/sgl_jax/srt/kernels/utils/perf.py`, which extracts
marker durations from profiler traces): CUDA events on the launching stream, warm-up first, the
L2 flushed between iterations by writing a buffer larger than it."""

from __future__ import annotations

import statistics
import time

import torch

_flush_buf: dict = {}


def flush_l2(device) -> None:
    buf = _flush_buf.get(str(device))
    if buf is None:
        buf = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=device)      # > 126 MB of L2
        _flush_buf[str(device)] = buf
    buf.zero_()


def multiple_iteration_timeit(fn, warmup: int = 3, iters: int = 10, flush: bool = True, device=None) -> dict:
    """Median / min / mean milliseconds of `fn()`."""
    if device is None:
        device = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
    device = torch.device(device)
    for _ in range(warmup):
        fn()
    times = []
    if device.type == "cuda":
        torch.cuda.synchronize(device)
        for _ in range(iters):
            if flush:
                flush_l2(device)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b))
    else:
        for _ in range(iters):
            t0 = time.perf_counter()
            fn()
            times.append((time.perf_counter() - t0) * 1e3)
    return {"median_ms": statistics.median(times), "min_ms": min(times), "mean_ms": statistics.fmean(times),
            "iters": iters}
