"""Bootstrap registry of prefill engines (reference
`python/sgl_jax/srt/disaggregation/bootstrap.py`: `build_app` :410, `BootstrapServer` :549,
`BootstrapClient` :639, `PrefillInfoCache` :867, `HeartbeatDaemon` :958, protocol floor :76,
compatibility check :112).

Prefill engines register `(engine_id, tp_rank) -> transfer address + KV layout` and keep the
entry alive with heartbeats; decode engines fetch the table, check that the KV layouts are
compatible with their own and cache it.  An entry whose heartbeat is older than `ttl` is
dropped, and with it the decode side stops routing pulls there."""

from __future__ import annotations

import logging
import threading
import time
from typing import Any

import requests
from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse

from . import pd_auth
from .common import metrics

logger = logging.getLogger(__name__)

PROTOCOL_VERSION = 3
MIN_PROTOCOL_VERSION = 2
DEFAULT_TTL = 15.0


class IncompatiblePeer(RuntimeError):
    pass


def check_compat(mine: dict, theirs: dict) -> None:
    """Raises `IncompatiblePeer` when two engines cannot exchange KV pages."""
    v = int(theirs.get("protocol_version", 0))
    if v < MIN_PROTOCOL_VERSION:
        raise IncompatiblePeer(f"peer speaks PD protocol {v}; this engine needs >= {MIN_PROTOCOL_VERSION}")
    for f in ("page_size", "num_layers", "page_bytes_per_layer", "dtype", "tp_size", "model"):
        if f in mine and f in theirs and mine[f] != theirs[f]:
            raise IncompatiblePeer(f"PD peers disagree on {f}: {mine[f]!r} vs {theirs[f]!r}")


# --------------------------------------------------------------------------- server
class Registry:
    """In-memory table behind the HTTP app (kept separate so it can be tested directly)."""

    def __init__(self, ttl: float = DEFAULT_TTL):
        self.ttl = ttl
        self.lock = threading.Lock()
        self.entries: dict[tuple[str, int], dict] = {}
        self.generation = 0

    def register(self, info: dict) -> dict:
        if int(info.get("protocol_version", 0)) < MIN_PROTOCOL_VERSION:
            raise IncompatiblePeer(f"protocol_version {info.get('protocol_version')} is below the floor "
                                   f"{MIN_PROTOCOL_VERSION}")
        key = (str(info["engine_id"]), int(info.get("tp_rank", 0)))
        with self.lock:
            for (eid, _), other in self.entries.items():
                if eid != key[0]:
                    check_compat(other, info)
                    break
            info = dict(info, last_heartbeat=time.time())
            fresh = key not in self.entries
            self.entries[key] = info
            if fresh:
                self.generation += 1
            metrics.set_registered_prefills(len(self.entries))
            return {"ok": True, "generation": self.generation, "ttl": self.ttl}

    def heartbeat(self, engine_id: str, tp_rank: int = 0) -> bool:
        with self.lock:
            e = self.entries.get((str(engine_id), int(tp_rank)))
            if e is None:
                return False
            e["last_heartbeat"] = time.time()
            return True

    def unregister(self, engine_id: str, tp_rank: int | None = None) -> int:
        with self.lock:
            keys = [k for k in self.entries if k[0] == str(engine_id) and (tp_rank is None or k[1] == int(tp_rank))]
            for k in keys:
                del self.entries[k]
            if keys:
                self.generation += 1
            metrics.set_registered_prefills(len(self.entries))
            return len(keys)

    def expire(self) -> int:
        now = time.time()
        with self.lock:
            dead = [k for k, e in self.entries.items() if now - e["last_heartbeat"] > self.ttl]
            for k in dead:
                logger.warning("bootstrap: prefill %s rank %d missed its heartbeats; dropped", *k)
                del self.entries[k]
            if dead:
                self.generation += 1
            metrics.set_registered_prefills(len(self.entries))
            return len(dead)

    def table(self) -> dict:
        self.expire()
        with self.lock:
            return {"generation": self.generation, "protocol_version": PROTOCOL_VERSION,
                    "prefills": [dict(e) for e in self.entries.values()]}


def build_app(registry: Registry | None = None, secret: str | None = None):
    reg = registry or Registry()
    app = FastAPI(title="sglang PD bootstrap")
    app.state.registry = reg

    def guard(request: Request):
        if not pd_auth.check_bearer(request.headers.get("authorization"), secret):
            return JSONResponse({"error": "unauthorized"}, status_code=401)
        return None

    @app.get("/health")
    async def health():
        return {"status": "ok", "protocol_version": PROTOCOL_VERSION}

    @app.post("/register")
    async def register(request: Request):
        if (r := guard(request)) is not None:
            return r
        try:
            return reg.register(await request.json())
        except IncompatiblePeer as e:
            return JSONResponse({"error": str(e)}, status_code=409)

    @app.post("/heartbeat")
    async def heartbeat(request: Request):
        if (r := guard(request)) is not None:
            return r
        b = await request.json()
        ok = reg.heartbeat(b["engine_id"], b.get("tp_rank", 0))
        return JSONResponse({"ok": ok}, status_code=200 if ok else 404)

    @app.post("/unregister")
    async def unregister(request: Request):
        if (r := guard(request)) is not None:
            return r
        b = await request.json()
        return {"removed": reg.unregister(b["engine_id"], b.get("tp_rank"))}

    @app.get("/prefills")
    async def prefills(request: Request):
        if (r := guard(request)) is not None:
            return r
        return reg.table()

    return app


class BootstrapServer:
    """Runs the registry app on a background thread."""

    def __init__(self, host: str = "127.0.0.1", port: int = 8998, ttl: float = DEFAULT_TTL, secret: str | None = None):
        import uvicorn
        self.registry = Registry(ttl)
        self.host, self.port = host, port
        self.app = build_app(self.registry, secret)
        self._server = uvicorn.Server(uvicorn.Config(self.app, host=host, port=port, log_level="error"))
        self._thread = threading.Thread(target=self._server.run, daemon=True, name="pd-bootstrap")

    @property
    def url(self) -> str:
        return f"http://{self.host}:{self.port}"

    def start(self, timeout: float = 10.0) -> "BootstrapServer":
        self._thread.start()
        t0 = time.time()
        while time.time() - t0 < timeout:
            try:
                if requests.get(self.url + "/health", timeout=0.5).status_code == 200:
                    return self
            except requests.RequestException:
                time.sleep(0.05)
        raise RuntimeError("bootstrap server did not come up")

    def stop(self):
        self._server.should_exit = True
        self._thread.join(timeout=5)


# --------------------------------------------------------------------------- clients
class BootstrapClient:
    def __init__(self, url: str, secret: str | None = None, timeout: float = 5.0):
        self.url = url.rstrip("/")
        self.headers = pd_auth.auth_headers(secret)
        self.timeout = timeout

    def _post(self, path: str, body: dict) -> requests.Response:
        return requests.post(self.url + path, json=body, headers=self.headers, timeout=self.timeout)

    def register(self, info: dict) -> dict:
        r = self._post("/register", dict(info, protocol_version=PROTOCOL_VERSION))
        if r.status_code == 409:
            raise IncompatiblePeer(r.json().get("error", "incompatible"))
        r.raise_for_status()
        return r.json()

    def heartbeat(self, engine_id: str, tp_rank: int = 0) -> bool:
        return self._post("/heartbeat", {"engine_id": engine_id, "tp_rank": tp_rank}).status_code == 200

    def unregister(self, engine_id: str, tp_rank: int | None = None) -> int:
        return self._post("/unregister", {"engine_id": engine_id, "tp_rank": tp_rank}).json().get("removed", 0)

    def prefills(self) -> dict:
        r = requests.get(self.url + "/prefills", headers=self.headers, timeout=self.timeout)
        r.raise_for_status()
        return r.json()


class PrefillInfoCache:
    """Decode-side view of the registry, refreshed at most every `refresh_interval` seconds
    (or at once after a miss)."""

    def __init__(self, client: BootstrapClient, my_layout: dict | None = None, refresh_interval: float = 2.0):
        self.client = client
        self.my_layout = my_layout or {}
        self.refresh_interval = refresh_interval
        self._table: dict[tuple[str, int], dict] = {}
        self._last = 0.0
        self._lock = threading.Lock()
        self.generation = -1

    def refresh(self, force: bool = False) -> None:
        with self._lock:
            if not force and time.time() - self._last < self.refresh_interval:
                return
            t = self.client.prefills()
            table = {}
            for e in t["prefills"]:
                try:
                    check_compat(self.my_layout, e)
                except IncompatiblePeer as ex:
                    logger.error("ignoring prefill %s: %s", e.get("engine_id"), ex)
                    continue
                table[(str(e["engine_id"]), int(e.get("tp_rank", 0)))] = e
            self._table = table
            self.generation = t["generation"]
            self._last = time.time()

    def lookup(self, engine_id: str | None = None, tp_rank: int = 0, room: int | None = None) -> dict | None:
        """The entry of `engine_id`, or — when no engine is named — one chosen by `room` so that
        a room always maps to the same prefill while the table does not change."""
        self.refresh()
        for attempt in range(2):
            with self._lock:
                if engine_id is not None:
                    e = self._table.get((str(engine_id), int(tp_rank)))
                else:
                    ids = sorted({k[0] for k in self._table})
                    e = self._table.get((ids[(room or 0) % len(ids)], int(tp_rank))) if ids else None
            if e is not None or attempt:
                return e
            self.refresh(force=True)
        return None

    def engines(self) -> list[str]:
        self.refresh()
        return sorted({k[0] for k in self._table})


class HeartbeatDaemon:
    """Keeps a prefill's registration alive; re-registers after the registry lost it
    (registry restart, missed beats)."""

    def __init__(self, client: BootstrapClient, info: dict, interval: float = 3.0):
        self.client, self.info, self.interval = client, info, interval
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True, name="pd-heartbeat")
        self.beats = 0
        self.reregistrations = 0

    def start(self) -> "HeartbeatDaemon":
        self.client.register(self.info)
        self._thread.start()
        return self

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                if self.client.heartbeat(self.info["engine_id"], self.info.get("tp_rank", 0)):
                    self.beats += 1
                else:
                    self.client.register(self.info)
                    self.reregistrations += 1
            except Exception as e:  # noqa: BLE001
                logger.warning("bootstrap heartbeat failed: %s", e)

    def stop(self, unregister: bool = True):
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=self.interval + 1)
        if unregister:
            try:
                self.client.unregister(self.info["engine_id"], self.info.get("tp_rank", 0))
            except Exception:  # noqa: BLE001
                pass
