"""Numerics tracing: per-layer activation statistics (min / max / mean / std / NaN / Inf counts, or the
full tensor) written as JSONL, switched at runtime through `/start_trace` `/stop_trace`
`/trace_status` (reference `python/sgl_jax/srt/precision_tracer.py:101-690`; the reference records
through `jax.pure_callback` inside the jitted model, here model code calls `precision_tracer.record`
directly — it is a no-op unless tracing is on, and it is skipped during CUDA-graph capture)."""

from __future__ import annotations

import json
import os
import threading
import time

import torch


class PrecisionTracer:
    def __init__(self):
        self.enabled = False
        self.output_file: str | None = None
        self.req_num: int | None = None
        self.save_tensor = False
        self.records = 0
        self.forward_id = 0
        self._lock = threading.Lock()
        self._fh = None

    def apply_state(self, state: dict):
        if state.get("enabled"):
            self.start_trace(state.get("output_file"), state.get("req_num"), bool(state.get("save_tensor")))
        else:
            self.stop_trace()

    def start_trace(self, output_file: str | None = None, req_num: int | None = None, save_tensor: bool = False):
        with self._lock:
            self.output_file = output_file or os.path.join(
                os.environ.get("SGLANG_PRECISION_TRACER_DIR", "/tmp"), f"precision_trace_{int(time.time())}.jsonl")
            os.makedirs(os.path.dirname(os.path.abspath(self.output_file)), exist_ok=True)
            self._fh = open(self.output_file, "a")
            self.req_num, self.save_tensor, self.records, self.enabled = req_num, save_tensor, 0, True

    def stop_trace(self) -> str | None:
        with self._lock:
            self.enabled = False
            if self._fh is not None:
                self._fh.close()
                self._fh = None
            return self.output_file

    def status(self) -> dict:
        return {"enabled": self.enabled, "output_file": self.output_file, "records": self.records}

    def begin_forward(self):
        self.forward_id += 1

    @staticmethod
    def _stats(t: torch.Tensor) -> dict:
        f = t.detach().float()
        finite = torch.isfinite(f)
        g = f[finite] if not bool(finite.all()) else f
        return {"shape": list(t.shape), "dtype": str(t.dtype), "min": float(g.min()) if g.numel() else None,
                "max": float(g.max()) if g.numel() else None, "mean": float(g.mean()) if g.numel() else None,
                "std": float(g.std()) if g.numel() > 1 else 0.0, "nan": int(torch.isnan(f).sum()),
                "inf": int(torch.isinf(f).sum())}

    def record(self, tensor: torch.Tensor, name: str, stage: str = "", layer_id: int | None = None):
        if not self.enabled or (tensor.is_cuda and torch.cuda.is_current_stream_capturing()):
            return
        rec = {"forward_id": self.forward_id, "name": name, "stage": stage, "layer_id": layer_id, **self._stats(tensor)}
        if self.save_tensor:
            rec["tensor"] = tensor.detach().float().cpu().flatten()[:4096].tolist()
        with self._lock:
            if self._fh is not None:
                self._fh.write(json.dumps(rec) + "\n")
                self._fh.flush()
                self.records += 1


precision_tracer = PrecisionTracer()


def trace_diff(file_a: str, file_b: str, rtol: float = 1e-2) -> list[dict]:
    """First records where two traces disagree (reference `python/sgl_jax/tools/trace_diff.py`)."""
    def load(p):
        with open(p) as f:
            return [json.loads(l) for l in f if l.strip()]
    out = []
    for a, b in zip(load(file_a), load(file_b)):
        if (a["name"], a["layer_id"]) != (b["name"], b["layer_id"]):
            out.append({"kind": "order", "a": a["name"], "b": b["name"]})
            break
        for k in ("mean", "std", "min", "max"):
            va, vb = a.get(k), b.get(k)
            if va is None or vb is None:
                continue
            if abs(va - vb) > rtol * max(abs(va), abs(vb), 1e-6):
                out.append({"kind": "value", "name": a["name"], "layer_id": a["layer_id"], "field": k, "a": va, "b": vb})
                break
    return out
