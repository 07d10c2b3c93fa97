"""Prometheus `pd_*` metrics (reference `python/sgl_jax/srt/disaggregation/common/metrics.py:50-88`).
Counters degrade to plain Python numbers when `prometheus_client` is unavailable, so the
values stay readable from tests and `/get_server_info`."""

from __future__ import annotations

import threading
from collections import defaultdict

_lock = threading.Lock()
_values: dict[tuple, float] = defaultdict(float)

try:  # pragma: no cover - exercised when the package is installed
    from prometheus_client import Counter, Gauge, Histogram
    _PROM = True
except Exception:  # noqa: BLE001
    _PROM = False

_metrics: dict[str, object] = {}


def _get(kind: str, name: str, doc: str, labels: tuple[str, ...]):
    if not _PROM:
        return None
    m = _metrics.get(name)
    if m is None:
        cls = {"counter": Counter, "gauge": Gauge, "hist": Histogram}[kind]
        try:
            m = cls(name, doc, labels)
        except ValueError:       # registered by another import of this module
            from prometheus_client import REGISTRY
            m = REGISTRY._names_to_collectors.get(name)
        _metrics[name] = m
    return m


def _bump(name: str, labels: dict, v: float = 1.0, kind: str = "counter", doc: str = ""):
    with _lock:
        key = (name, tuple(sorted(labels.items())))
        if kind == "gauge":
            _values[key] = v
        else:
            _values[key] += v
    m = _get(kind, name, doc or name, tuple(sorted(labels)))
    if m is not None:
        try:
            h = m.labels(**labels) if labels else m
            if kind == "counter":
                h.inc(v)
            elif kind == "gauge":
                h.set(v)
            else:
                h.observe(v)
        except Exception:  # noqa: BLE001
            pass


def count_transition(frm: str, to: str, role: str):
    _bump("pd_state_transition_total", {"from_state": frm, "to_state": to, "role": role},
          doc="KV transfer state transitions")


def count_transfer(role: str, outcome: str, nbytes: int = 0, seconds: float | None = None):
    _bump("pd_transfer_total", {"role": role, "outcome": outcome}, doc="finished KV transfers")
    if nbytes:
        _bump("pd_transfer_bytes_total", {"role": role}, nbytes, doc="KV bytes moved")
    if seconds is not None:
        _bump("pd_transfer_seconds", {"role": role}, seconds, kind="hist", doc="KV transfer latency")


def count_reaped(role: str, reason: str):
    _bump("pd_reaped_total", {"role": role, "reason": reason}, doc="transfers ended by the timeout reaper")


def set_queue_depth(queue: str, depth: int):
    _bump("pd_queue_depth", {"queue": queue}, depth, kind="gauge", doc="PD scheduler queue depth")


def set_registered_prefills(n: int):
    _bump("pd_bootstrap_registered_prefills", {}, n, kind="gauge", doc="live prefill registrations")


def snapshot() -> dict:
    with _lock:
        return {f"{n}{dict(l) if l else ''}": v for (n, l), v in _values.items()}


def reset():
    with _lock:
        _values.clear()
