"""Pull-done acknowledgements from decode back to prefill (reference
`python/sgl_jax/srt/disaggregation/common/zmq_notifier.py`): once a decode engine holds the KV
it tells the prefill engine, which may then release the pages.  Messages carry an HMAC tag
when a shared secret is configured."""

from __future__ import annotations

import json
import logging
import threading
from typing import Callable

from .. import pd_auth

logger = logging.getLogger(__name__)


class AckListener:
    """Prefill side: PULL socket + callback thread."""

    def __init__(self, host: str, port: int, on_ack: Callable[[str, bool, str], None], secret: str | None = None):
        import zmq
        self._ctx = zmq.Context.instance()
        self._sock = self._ctx.socket(zmq.PULL)
        self._sock.setsockopt(zmq.LINGER, 0)
        self.port = port or self._sock.bind_to_random_port(f"tcp://{host}")
        if port:
            self._sock.bind(f"tcp://{host}:{port}")
        self.addr = f"{host}:{self.port}"
        self.on_ack = on_ack
        self.secret = secret
        self.rejected = 0
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True, name="pd-ack")
        self._thread.start()

    def _run(self):
        import zmq
        poller = zmq.Poller()
        poller.register(self._sock, zmq.POLLIN)
        while not self._stop.is_set():
            if not poller.poll(100):
                continue
            try:
                tag, body = self._sock.recv_multipart()
            except Exception:  # noqa: BLE001
                continue
            if not pd_auth.verify(body, tag, self.secret):
                self.rejected += 1
                logger.warning("dropped an unauthenticated PD acknowledgement")
                continue
            m = json.loads(body)
            try:
                self.on_ack(m["transfer_id"], bool(m.get("ok", True)), m.get("reason", ""))
            except Exception:  # noqa: BLE001
                logger.exception("ack callback failed")

    def stop(self):
        self._stop.set()
        self._thread.join(timeout=2)
        self._sock.close()


class AckSender:
    """Decode side: one PUSH socket per prefill peer, created lazily."""

    def __init__(self, secret: str | None = None):
        import zmq
        self._ctx = zmq.Context.instance()
        self._socks: dict[str, object] = {}
        self._lock = threading.Lock()
        self.secret = secret

    def send(self, addr: str, transfer_id: str, ok: bool = True, reason: str = ""):
        import zmq
        body = json.dumps({"transfer_id": transfer_id, "ok": ok, "reason": reason}).encode()
        with self._lock:
            s = self._socks.get(addr)
            if s is None:
                s = self._ctx.socket(zmq.PUSH)
                s.setsockopt(zmq.LINGER, 500)
                s.connect(f"tcp://{addr}")
                self._socks[addr] = s
            s.send_multipart([pd_auth.sign(body, self.secret), body])

    def close(self):
        with self._lock:
            for s in self._socks.values():
                s.close()
            self._socks.clear()
