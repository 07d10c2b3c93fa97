"""Device-memory accounting helpers (reference `python/sgl_jax/srt/memory_profiler.py`): a decorator /
context manager that logs allocated-bytes deltas, per-module parameter sizes, and snapshot dumps to
`SGL_MEMORY_OUTPUT_DIR`."""

from __future__ import annotations

import contextlib
import functools
import json
import os
import time

import torch


def _allocated(device=None) -> int:
    return torch.cuda.memory_allocated(device) if torch.cuda.is_available() else 0


class MemoryProfiler:
    def __init__(self):
        self.enabled = os.environ.get("SGL_MEMORY_PROFILE", "0") == "1"
        self.output_dir = os.environ.get("SGL_MEMORY_OUTPUT_DIR", "/tmp/sgl_memory")
        self.events: list[dict] = []

    @contextlib.contextmanager
    def scope(self, name: str):
        if not self.enabled:
            yield
            return
        before, t0 = _allocated(), time.time()
        try:
            yield
        finally:
            after = _allocated()
            self.events.append({"name": name, "delta_mb": (after - before) / 2 ** 20, "after_mb": after / 2 ** 20,
                                "peak_mb": (torch.cuda.max_memory_allocated() / 2 ** 20) if torch.cuda.is_available() else 0,
                                "seconds": time.time() - t0})

    def profile(self, name: str | None = None):
        def deco(fn):
            @functools.wraps(fn)
            def wrapper(*a, **k):
                with self.scope(name or fn.__qualname__):
                    return fn(*a, **k)
            return wrapper
        return deco

    @staticmethod
    def module_sizes(model: torch.nn.Module, depth: int = 2) -> dict[str, float]:
        out: dict[str, float] = {}
        for n, p in model.named_parameters():
            key = ".".join(n.split(".")[:depth])
            out[key] = out.get(key, 0.0) + p.numel() * p.element_size() / 2 ** 20
        return out

    def report(self, tag: str = "memory") -> str:
        os.makedirs(self.output_dir, exist_ok=True)
        path = os.path.join(self.output_dir, f"{tag}_{int(time.time())}.json")
        with open(path, "w") as f:
            json.dump(self.events, f, indent=1)
        return path

    def snapshot(self, tag: str = "snapshot") -> str | None:
        if not torch.cuda.is_available():
            return None
        os.makedirs(self.output_dir, exist_ok=True)
        path = os.path.join(self.output_dir, f"{tag}_{int(time.time())}.txt")
        with open(path, "w") as f:
            f.write(torch.cuda.memory_summary())
        return path


memory_profiler = MemoryProfiler()
memory_profile = memory_profiler.profile
profile_memory_scope = memory_profiler.scope
