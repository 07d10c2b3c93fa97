"""The KV manager shared by both roles: senders / receivers over a transfer backend, a pool of
pull workers, the timeout reaper and graceful drain (reference
`python/sgl_jax/srt/disaggregation/common/core.py`: `CommonKVManager` :25, reaper :140-203,
drain :211)."""

from __future__ import annotations

import logging
import queue
import threading
import time

import numpy as np

from ..base.kv_manager import KVManager, KVPoll, KVReceiver, KVSender, StateHolder
from . import metrics
from .zmq_notifier import AckListener, AckSender

logger = logging.getLogger(__name__)


class CommonKVSender(KVSender):
    def __init__(self, mgr: "CommonKVManager", req_id: str):
        self.mgr, self.req_id = mgr, req_id
        self.state = StateHolder("prefill")
        self.transfer_id: str | None = None
        self.pages = None
        self.meta: dict = {}
        self.t_send = 0.0

    def init(self, kv_pages, transfer_id: str, first_token: int | None = None, meta: dict | None = None) -> None:
        self.pages = np.asarray(kv_pages, np.int64)
        self.transfer_id = transfer_id
        self.meta = dict(meta or {}, first_token=first_token, ack_addr=self.mgr.ack_addr)
        self.state.transition(KVPoll.WAITING_FOR_INPUT)

    def send(self) -> None:
        """Publish the pages; the transfer completes when the decode side acknowledges."""
        self.mgr.backend.register(self.transfer_id, self.pages, self.meta)
        if self.mgr.mirror is not None:
            self.mgr.mirror.register(self.transfer_id, self.pages, self.meta)
        self.t_send = time.monotonic()
        self.state.transition(KVPoll.TRANSFERRING)
        self.mgr._track_sender(self)

    def poll(self) -> KVPoll:
        return self.state.state

    def _on_ack(self, ok: bool, reason: str):
        if self.state.state.terminal:
            return
        if ok:
            self.state.transition(KVPoll.SUCCESS)
            nbytes = len(self.pages) * self.mgr.page_bytes
            metrics.count_transfer("prefill", "success", nbytes, time.monotonic() - self.t_send)
        else:
            self.state.fail(reason or "decode reported a failed pull")
            metrics.count_transfer("prefill", "failed")
        self.mgr.backend.unregister(self.transfer_id)

    def abort(self) -> None:
        self.state.fail("aborted")
        if self.transfer_id:
            self.mgr.backend.unregister(self.transfer_id)

    def clear(self) -> None:
        self.mgr._forget_sender(self)


class CommonKVReceiver(KVReceiver):
    def __init__(self, mgr: "CommonKVManager", req_id: str):
        self.mgr, self.req_id = mgr, req_id
        self.state = StateHolder("decode")
        self.transfer_id: str | None = None
        self.dst_pages = None
        self.prefill_addr: str | None = None
        self.meta: dict | None = None
        self.t_start = 0.0

    def init(self, dst_pages, transfer_id: str, prefill_addr: str) -> None:
        self.dst_pages = np.asarray(dst_pages, np.int64)
        self.transfer_id = transfer_id
        self.prefill_addr = prefill_addr
        self.state.transition(KVPoll.WAITING_FOR_INPUT)
        self.t_start = time.monotonic()
        self.mgr._submit_pull(self)

    def _run(self):
        if self.state.state.terminal:
            return
        self.state.transition(KVPoll.TRANSFERRING)
        mirror = self.mgr.mirror
        try:
            if mirror is not None:
                # the follower ranks pull their shards from the prefill ranks of the same index meanwhile
                mirror.pull(self.transfer_id, self.dst_pages, self.mgr.backend.query_peers(self.prefill_addr))
            self.meta = self.mgr.backend.pull(self.prefill_addr, self.transfer_id, self.dst_pages)
            if mirror is not None:
                bad = mirror.wait(self.transfer_id)
                if bad:
                    raise RuntimeError(bad)
        except Exception as e:  # noqa: BLE001
            if mirror is not None:
                mirror.drop(self.transfer_id)
            self.state.fail(str(e))
            metrics.count_transfer("decode", "failed")
            self._ack(False, str(e))
            return
        if self.state.state.terminal:       # reaped / aborted while the pull ran
            self._ack(False, self.state.failure or "aborted")
            return
        self.state.transition(KVPoll.SUCCESS)
        metrics.count_transfer("decode", "success", len(self.dst_pages) * self.mgr.page_bytes,
                               time.monotonic() - self.t_start)
        self._ack(True, "")

    def _ack(self, ok: bool, reason: str):
        addr = (self.meta or {}).get("ack_addr") or self.mgr.ack_addr_of(self.prefill_addr)
        if addr:
            try:
                self.mgr.ack_sender.send(addr, self.transfer_id, ok, reason)
            except Exception:  # noqa: BLE001
                logger.exception("could not acknowledge %s", self.transfer_id)

    def poll(self) -> KVPoll:
        return self.state.state

    def abort(self) -> None:
        self.state.fail("aborted")

    def clear(self) -> None:
        self.mgr._forget_receiver(self)


class CommonKVManager(KVManager):
    def __init__(self, role: str, backend, page_bytes: int, host: str = "127.0.0.1", side_channel_port: int = 0,
                 secret: str | None = None, num_pull_workers: int = 4, pull_timeout: float = 30.0,
                 ack_timeout: float = 60.0, reaper_interval: float = 5.0, mirror=None):
        assert role in ("prefill", "decode")
        self.mirror = mirror      # `tp_mirror.RankMirror` when the engine has more than one tensor rank
        self.role, self.backend, self.page_bytes = role, backend, page_bytes
        self.pull_timeout, self.ack_timeout = pull_timeout, ack_timeout
        self.senders: dict[str, CommonKVSender] = {}
        self.receivers: dict[str, CommonKVReceiver] = {}
        self.lock = threading.Lock()
        self.draining = False
        self._stop = threading.Event()
        self.ack_listener = None
        self.ack_addr = None
        self.ack_sender = AckSender(secret)
        self._ack_addrs: dict[str, str] = {}
        if role == "prefill":
            self.ack_listener = AckListener(host, side_channel_port, self._on_ack, secret)
            self.ack_addr = self.ack_listener.addr
        self._q: "queue.Queue[CommonKVReceiver | None]" = queue.Queue()
        self._workers = []
        if role == "decode":
            for i in range(max(1, num_pull_workers)):
                t = threading.Thread(target=self._pull_worker, daemon=True, name=f"pd-pull-{i}")
                t.start()
                self._workers.append(t)
        self.reaper_interval = reaper_interval
        self._reaper = threading.Thread(target=self._reap_loop, daemon=True, name="pd-reaper")
        self._reaper.start()

    # ------------------------------------------------------------------ factory
    def create_sender(self, req_id: str) -> CommonKVSender:
        if self.draining:
            raise RuntimeError("KV manager is draining; no new transfers")
        return CommonKVSender(self, req_id)

    def create_receiver(self, req_id: str) -> CommonKVReceiver:
        if self.draining:
            raise RuntimeError("KV manager is draining; no new transfers")
        r = CommonKVReceiver(self, req_id)
        return r

    def set_ack_addr(self, prefill_addr: str, ack_addr: str):
        self._ack_addrs[prefill_addr] = ack_addr

    def ack_addr_of(self, prefill_addr: str) -> str | None:
        return self._ack_addrs.get(prefill_addr)

    # ------------------------------------------------------------------ bookkeeping
    def _track_sender(self, s: CommonKVSender):
        with self.lock:
            self.senders[s.transfer_id] = s

    def _forget_sender(self, s: CommonKVSender):
        with self.lock:
            self.senders.pop(s.transfer_id, None)
        if s.transfer_id:
            self.backend.unregister(s.transfer_id)
            if self.mirror is not None:
                # runs on the scheduler thread, before the request's pages are released
                self.mirror.unregister(s.transfer_id)

    def _forget_receiver(self, r: CommonKVReceiver):
        with self.lock:
            self.receivers.pop(r.transfer_id, None)

    def _on_ack(self, transfer_id: str, ok: bool, reason: str):
        with self.lock:
            s = self.senders.get(transfer_id)
        if s is not None:
            s._on_ack(ok, reason)

    def _submit_pull(self, r: CommonKVReceiver):
        with self.lock:
            self.receivers[r.transfer_id] = r
        self._q.put(r)

    def _pull_worker(self):
        while True:
            r = self._q.get()
            if r is None:
                return
            try:
                r._run()
            except Exception:  # noqa: BLE001
                logger.exception("pull worker crashed on %s", r.transfer_id)
                r.state.fail("pull worker error")

    # ------------------------------------------------------------------ reaper
    def reap_once(self) -> int:
        """Fail transfers whose peer went silent: a sender nobody acknowledged within
        `ack_timeout`, a receiver that has not finished within `pull_timeout` (+ slack)."""
        n = 0
        with self.lock:
            senders = list(self.senders.values())
            receivers = list(self.receivers.values())
        for s in senders:
            if s.state.state == KVPoll.TRANSFERRING and s.state.age() > self.ack_timeout:
                s.state.fail(f"no acknowledgement within {self.ack_timeout}s")
                self.backend.unregister(s.transfer_id)
                metrics.count_reaped("prefill", "ack_timeout")
                n += 1
        for r in receivers:
            if not r.state.state.terminal and r.state.age() > self.pull_timeout + 5.0:
                r.state.fail(f"pull did not finish within {self.pull_timeout}s")
                metrics.count_reaped("decode", "pull_timeout")
                n += 1
        return n

    def _reap_loop(self):
        while not self._stop.wait(self.reaper_interval):
            try:
                self.reap_once()
            except Exception:  # noqa: BLE001
                logger.exception("reaper iteration failed")

    # ------------------------------------------------------------------ shutdown
    def inflight(self) -> int:
        with self.lock:
            return sum(not s.state.state.terminal for s in self.senders.values()) + \
                sum(not r.state.state.terminal for r in self.receivers.values())

    def drain(self, timeout: float = 30.0) -> bool:
        """Stop taking new transfers and wait for the running ones; True when none is left."""
        self.draining = True
        t0 = time.monotonic()
        while self.inflight() and time.monotonic() - t0 < timeout:
            time.sleep(0.02)
        return self.inflight() == 0

    def shutdown(self):
        self._stop.set()
        for _ in self._workers:
            self._q.put(None)
        if self.ack_listener is not None:
            self.ack_listener.stop()
        self.ack_sender.close()
        if self.mirror is not None:
            self.mirror.stop()
        if hasattr(self.backend, "stop"):
            self.backend.stop()
