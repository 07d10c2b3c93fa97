"""KV hand-over for every tensor-parallel rank of a prefill / decode pair.

Each tensor rank holds the KV heads of its shard, so a request's pages have to travel once per rank: prefill
rank r -> decode rank r (the reference's `disaggregation/jax_transfer/conn.py` moves every shard of the gathered
array the same way).  Rank 0 of each engine runs the scheduler and the existing transfer manager; the ranks
behind it are driven through the step channel:

* prefill followers run their own transfer server over their own pool; rank 0 tells them which pages to
  publish under which transfer id (`pd_register`) and when to forget them (`pd_unregister`);
* decode followers pull from the prefill rank of the same index when told (`pd_pull`), on a small thread pool,
  and report the outcome to rank 0 through an *uplink* socket (followers -> rank 0, one PUSH per message);
* rank 0 of the decode engine acknowledges the transfer to the prefill engine only after its own pull and all
  followers' pulls have finished, so no rank's pages are released while a peer still reads them.

Control messages share the ordered channel of the step batches: a follower has launched the prefill of a request
before it is asked to publish its pages, and has finished its pull before any batch uses the request (rank 0
admits it only after every rank reported).
"""

from __future__ import annotations

import json
import logging
import threading
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from . import pd_auth

logger = logging.getLogger(__name__)


class Uplink:
    """Rank 0's inbox for its follower ranks: transfer addresses at start-up, pull outcomes later."""

    def __init__(self, host: str = "127.0.0.1", secret: str | None = None):
        import zmq
        self.secret = secret
        self._ctx = zmq.Context.instance()
        self._sock = self._ctx.socket(zmq.PULL)
        self._sock.setsockopt(zmq.LINGER, 0)
        port = self._sock.bind_to_random_port(f"tcp://{host}")
        self.addr = f"{host}:{port}"
        self.addrs: dict[int, str] = {}
        self.done: dict[str, dict[int, str]] = {}      # transfer id -> {rank: "" (ok) | reason}
        self.dropped: set[str] = set()                 # transfers rank 0 gave up; late reports are ignored
        self.cv = threading.Condition()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._serve, daemon=True, name="pd-uplink")
        self._thread.start()

    def _serve(self):
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
                continue
            m = json.loads(body)
            with self.cv:
                if m["kind"] == "addr":
                    self.addrs[int(m["rank"])] = m["addr"]
                elif m["kind"] == "done" and m["transfer_id"] in self.dropped:
                    pass                                   # rank 0 already gave this transfer up
                elif m["kind"] == "done":
                    self.done.setdefault(m["transfer_id"], {})[int(m["rank"])] = "" if m["ok"] else (m.get("reason") or "failed")
                self.cv.notify_all()

    def wait_addrs(self, n: int, timeout: float = 60.0) -> list[str]:
        with self.cv:
            ok = self.cv.wait_for(lambda: len(self.addrs) >= n, timeout)
        if not ok:
            raise RuntimeError(f"only {len(self.addrs)} of {n} follower ranks reported a transfer address")
        return [self.addrs[r] for r in sorted(self.addrs)]

    def wait_done(self, transfer_id: str, n: int, timeout: float) -> str:
        """'' when `n` followers finished their pull, else the first failure (or a time-out message)."""
        with self.cv:
            ok = self.cv.wait_for(lambda: len(self.done.get(transfer_id, {})) >= n
                                  or any(self.done.get(transfer_id, {}).values()), timeout)
            got = self.done.pop(transfer_id, {})
        bad = [f"rank {r}: {v}" for r, v in sorted(got.items()) if v]
        if bad:
            return bad[0]
        return "" if ok else f"{n - len(got)} follower rank(s) did not finish their pull within {timeout:.0f}s"

    def drop(self, transfer_id: str):
        with self.cv:
            self.done.pop(transfer_id, None)
            if len(self.dropped) > 4096:
                self.dropped.clear()
            self.dropped.add(transfer_id)

    def stop(self):
        self._stop.set()
        self._thread.join(timeout=2)
        try:
            self._sock.close()
        except Exception:  # noqa: BLE001
            pass


def _push(addr: str, secret, msg: dict):
    import zmq
    s = zmq.Context.instance().socket(zmq.PUSH)
    s.setsockopt(zmq.LINGER, 2000)
    s.connect(f"tcp://{addr}")
    body = json.dumps(msg).encode()
    try:
        s.send_multipart([pd_auth.sign(body, secret), body])
    finally:
        s.close()


class FollowerTransfer:
    """What a follower rank holds: a transfer backend over its own KV pool and a few pull threads."""

    def __init__(self, worker, cfg: dict):
        from .transfer.zmq_transfer import ZmqTransferBackend
        self.rank = worker.tp_rank
        self.secret = cfg.get("secret")
        self.uplink = cfg["uplink"]
        self.device = worker.device
        self.backend = ZmqTransferBackend(worker.model_runner.token_to_kv_pool, cfg.get("host", "127.0.0.1"), 0,
                                          cfg.get("mode", "tcp"), self.secret, cfg.get("pull_timeout", 30.0))
        self.pool = ThreadPoolExecutor(max_workers=max(1, int(cfg.get("workers", 2))), thread_name_prefix="pd-follower-pull")
        if cfg["role"] == "prefill":
            _push(self.uplink, self.secret, {"kind": "addr", "rank": self.rank, "addr": self.backend.start()})

    def handle(self, kind: str, p: dict):
        if kind == "pd_register":
            self.backend.register(p["transfer_id"], np.asarray(p["pages"], np.int64), p.get("meta") or {})
        elif kind == "pd_unregister":
            self.backend.unregister(p["transfer_id"])
        elif kind == "pd_pull":
            self.pool.submit(self._pull, p["transfer_id"], p["addrs"][self.rank], np.asarray(p["pages"], np.int64))
        elif kind == "pd_stop":
            self.stop()

    def _pull(self, tid: str, addr: str, pages: np.ndarray):
        ok, reason = True, ""
        try:
            if getattr(self.device, "type", "cpu") == "cuda":
                import torch
                torch.cuda.set_device(self.device)
            self.backend.pull(addr, tid, pages)
        except Exception as e:  # noqa: BLE001
            ok, reason = False, str(e)
        try:
            _push(self.uplink, self.secret, {"kind": "done", "rank": self.rank, "transfer_id": tid, "ok": ok, "reason": reason})
        except Exception:  # noqa: BLE001
            logger.exception("could not report the pull of %s", tid)

    def stop(self):
        self.pool.shutdown(wait=False)
        if self.backend._thread is not None:
            self.backend.stop()


def handle_follower_control(worker, kind: str, payload: dict) -> None:
    """Entry for the follower loop (`managers/tp_worker.py`): `pd_init` builds the rank's transfer state, the
    other `pd_*` messages use it."""
    if kind == "pd_init":
        worker.pd_transfer = FollowerTransfer(worker, payload)
        return
    ft = getattr(worker, "pd_transfer", None)
    if ft is None:
        logger.error("%s before pd_init", kind)
        return
    ft.handle(kind, payload)


class RankMirror:
    """Rank 0's side: fan the bookkeeping of a transfer out to the follower ranks."""

    def __init__(self, worker, role: str, host: str, secret, mode: str, pull_timeout: float, own_addr: str | None):
        self.worker, self.role = worker, role
        self.n = worker.tp_size - 1
        self.pull_timeout = pull_timeout
        self.uplink = Uplink(host, secret)
        worker.send_control("pd_init", {"role": role, "uplink": self.uplink.addr, "secret": secret, "host": host,
                                        "mode": mode, "pull_timeout": pull_timeout})
        # prefill: the transfer address of every rank, rank 0 first
        self.addrs = [own_addr] + self.uplink.wait_addrs(self.n) if role == "prefill" else None

    # prefill
    def register(self, transfer_id: str, pages, meta: dict):
        self.worker.send_control("pd_register", {"transfer_id": transfer_id, "pages": np.asarray(pages).tolist(),
                                                 "meta": {"rid": meta.get("rid")}})

    def unregister(self, transfer_id: str):
        self.worker.send_control("pd_unregister", {"transfer_id": transfer_id})

    # decode
    def pull(self, transfer_id: str, pages, addrs: list[str]):
        if len(addrs) != self.n + 1:
            raise RuntimeError(f"the prefill engine runs {len(addrs)} tensor ranks, this engine {self.n + 1}")
        self.worker.send_control("pd_pull", {"transfer_id": transfer_id, "pages": np.asarray(pages).tolist(), "addrs": addrs})

    def wait(self, transfer_id: str) -> str:
        return self.uplink.wait_done(transfer_id, self.n, self.pull_timeout + 5.0)

    def drop(self, transfer_id: str):
        self.uplink.drop(transfer_id)

    def stop(self):
        try:
            self.worker.send_control("pd_stop", {})
        except Exception:  # noqa: BLE001
            pass
        self.uplink.stop()
