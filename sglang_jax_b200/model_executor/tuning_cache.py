"""Measured kernel plans, persisted on disk.

The reference avoids paying for compilation twice with a persistent XLA compile cache and an optional
ahead-of-time executable cache (`python/sgl_jax/srt/model_executor/aot_dispatch.py`, `SGLANG_JAX_AOT_DISPATCH`),
and ships tables of tuned block sizes per kernel and device.  Kernels here are compiled ahead of time and CUDA
graphs cannot be serialised, so what is worth keeping between runs is the *plan*: for every decode-sized GEMM
shape of the model, which candidate is fastest on this GPU: the tcgen05 kernel with tokens on the MMA M dimension
(0), with weight rows on M and stream-K (1), the library GEMM (2: plain projections only; the fused
GEMM + collective kernels are not part of the choice), or the cluster split-K kernel of `csrc/gemm_decode_cluster.cu`
(3: up to 128 tokens).  With `SGLB_GEMM_AUTOTUNE=1` the first engine start measures
each shape it meets (a few launches per candidate with the L2 flushed in between, CUDA events, median) before the
decode graphs are captured, and stores
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
        self._flush = None
        # SGLB_GEMM_PLAN_LIBRARY=0 keeps the choice among this library's own kernels
        self.candidates = (0, 1, 2) if os.environ.get("SGLB_GEMM_PLAN_LIBRARY", "1") == "1" else (0, 1)
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

    def mode_for(self, M: int, N: int, K: int, run, extra: tuple = ()) -> int:
        """Candidate for a decode-sized GEMM (-1 = the launcher's default).  `run(mode)` launches the GEMM once with
        that candidate on the current stream; it is only called for shapes not in the table, and never while a graph
        is being captured.  `extra`: further candidates the caller can run for this shape."""
        b = _bucket(M)
        if b == 0:
            return -1
        key = f"{b}x{N}x{K}"
        allowed = tuple(self.candidates) + tuple(extra)
        mode = self.table.get(key)
        if mode is not None and mode in allowed:
            return mode                 # (an entry for a candidate that is switched off here is measured again)
        if not self.measure or torch.cuda.is_current_stream_capturing():
            return -1
        times = {}
        if self._flush is None:
            # weights come from HBM in a real step (every layer has its own): measure with a cold L2
            with torch.inference_mode(False):      # a plain tensor: it is written in and out of inference mode
                self._flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")
        for cand in allowed:
            for _ in range(2):
                run(cand)
            ts = []
            for _ in range(5):
                self._flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                run(cand)
                e1.record()
                e1.synchronize()
                ts.append(e0.elapsed_time(e1))
            times[cand] = sorted(ts)[len(ts) // 2]
        mode = min(times, key=times.get)
        self.table[key] = mode
        self.dirty = True
        self.measured += 1
        return mode

    def save(self):
        self._flush = None
        if not (self.path and self.dirty):
            return
        os.makedirs(os.path.dirname(self.path), exist_ok=True)
        tmp = self.path + f".{os.getpid()}.tmp"
        with open(tmp, "w") as f:
            json.dump({"gemm_mode": self.table}, f, indent=1, sort_keys=True)
        os.replace(tmp, self.path)
        self.dirty = False
        logger.info("saved %d tuned GEMM shapes to %s", len(self.table), self.path)
