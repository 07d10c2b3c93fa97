"""Measured kernel plans, persisted on disk.

The reference avoids paying for compilation twice with a persistent XLA compile cache and an optional
ahead-of-time executable cache (`python/sgl_jax/srt/model_executor/aot_dispatch.py`, `SGLANG_JAX_AOT_DISPATCH`),
and ships tables of tuned block sizes per kernel and device.  Kernels here are compiled ahead of time and CUDA
graphs cannot be serialised, so what is worth keeping between runs is the *plan*: for every decode-sized GEMM
shape of the model, which operand assignment of the tcgen05 kernel is faster on this GPU (tokens on the MMA M
dimension with stream-K, or weight rows on M).  With `SGLB_GEMM_AUTOTUNE=1` the first engine start measures each
shape it meets (a few launches per candidate, CUDA events) before the decode graphs are captured, and stores
the table under `SGLB_TUNING_CACHE_DIR` (default `~/.cache/sglang_jax_b200`), keyed by GPU name and by a digest
of the kernel library; later starts load it and measure nothing.
"""

from __future__ import annotations

import hashlib
import json
import logging
import os

import torch

logger = logging.getLogger(__name__)

_M_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def _bucket(m: int) -> int:
    for b in _M_BUCKETS:
        if m <= b:
            return b
    return 0


class GemmPlan:
    def __init__(self, path: str | None = None, measure: bool = True):
        self.path = path
        self.measure = measure
        self.table: dict[str, int] = {}
        self.dirty = False
        self.measured = 0
        if path and os.path.exists(path):
            try:
                with open(path) as f:
                    self.table = {k: int(v) for k, v in json.load(f).get("gemm_mode", {}).items()}
                logger.info("loaded %d tuned GEMM shapes from %s", len(self.table), path)
            except Exception as e:
                logger.warning("ignoring unreadable tuning cache %s: %s", path, e)

    @staticmethod
    def default_path(lib_path: str) -> str:
        root = os.environ.get("SGLB_TUNING_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "sglang_jax_b200")
        gpu = torch.cuda.get_device_name(0).replace(" ", "_") if torch.cuda.is_available() else "cpu"
        h = hashlib.sha256()
        with open(lib_path, "rb") as f:
            h.update(f.read())
        return os.path.join(root, f"tuning_{gpu}_{h.hexdigest()[:12]}.json")

    def mode_for(self, M: int, N: int, K: int, run) -> int:
        """Operand assignment for a decode-sized GEMM (-1 = the launcher's default).  `run(mode)` launches the GEMM
        once with that assignment on the current stream; it is only called for shapes not in the table, and never
        while a graph is being captured."""
        b = _bucket(M)
        if b == 0:
            return -1
        key = f"{b}x{N}x{K}"
        mode = self.table.get(key)
        if mode is not None:
            return mode
        if not self.measure or torch.cuda.is_current_stream_capturing():
            return -1
        times = {}
        for cand in (0, 1):
            for _ in range(2):
                run(cand)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                run(cand)
            e1.record()
            e1.synchronize()
            times[cand] = e0.elapsed_time(e1)
        mode = min(times, key=times.get)
        self.table[key] = mode
        self.dirty = True
        self.measured += 1
        return mode

    def save(self):
        if not (self.path and self.dirty):
            return
        os.makedirs(os.path.dirname(self.path), exist_ok=True)
        tmp = self.path + f".{os.getpid()}.tmp"
        with open(tmp, "w") as f:
            json.dump({"gemm_mode": self.table}, f, indent=1, sort_keys=True)
        os.replace(tmp, self.path)
        self.dirty = False
        logger.info("saved %d tuned GEMM shapes to %s", len(self.table), self.path)
