"""The contract between the schedulers and a KV transfer backend (reference
`python/sgl_jax/srt/disaggregation/base/kv_manager.py:22-137`).

A request's transfer walks BOOTSTRAPPING -> WAITING_FOR_INPUT -> TRANSFERRING -> SUCCESS, and
may drop to FAILED from any non-terminal state; anything else is a bug and raises."""

from __future__ import annotations

import abc
import enum
import time


class KVPoll(enum.Enum):
    BOOTSTRAPPING = "bootstrapping"
    WAITING_FOR_INPUT = "waiting_for_input"
    TRANSFERRING = "transferring"
    SUCCESS = "success"
    FAILED = "failed"

    @property
    def terminal(self) -> bool:
        return self in (KVPoll.SUCCESS, KVPoll.FAILED)


_ORDER = [KVPoll.BOOTSTRAPPING, KVPoll.WAITING_FOR_INPUT, KVPoll.TRANSFERRING, KVPoll.SUCCESS]


def is_legal_transition(cur: KVPoll, nxt: KVPoll) -> bool:
    if cur.terminal:
        return False
    if nxt == KVPoll.FAILED:
        return True
    return _ORDER.index(nxt) == _ORDER.index(cur) + 1


class StateHolder:
    """State + timestamps of one transfer; every change goes through `transition`."""

    def __init__(self, role: str | None = None, initial: KVPoll = KVPoll.BOOTSTRAPPING):
        self.role = role
        self._state = initial
        self.created = time.monotonic()
        self.last_change = self.created
        self.failure: str | None = None

    @property
    def state(self) -> KVPoll:
        return self._state

    def transition(self, nxt: KVPoll, reason: str | None = None) -> None:
        if not is_legal_transition(self._state, nxt):
            raise ValueError(f"illegal KVPoll transition: {self._state.value} -> {nxt.value}")
        prev, self._state = self._state, nxt
        self.last_change = time.monotonic()
        if nxt == KVPoll.FAILED:
            self.failure = reason or "transfer failed"
        if self.role is not None:
            from ..common.metrics import count_transition
            count_transition(prev.value, nxt.value, self.role)

    def fail(self, reason: str) -> None:
        if not self._state.terminal:
            self.transition(KVPoll.FAILED, reason)

    def age(self) -> float:
        return time.monotonic() - self.last_change


class KVSender(abc.ABC):
    """Prefill side, one per request."""

    @abc.abstractmethod
    def init(self, kv_pages, transfer_id: str, first_token: int | None = None, meta: dict | None = None) -> None: ...

    @abc.abstractmethod
    def send(self) -> None: ...

    @abc.abstractmethod
    def poll(self) -> KVPoll: ...

    @abc.abstractmethod
    def abort(self) -> None: ...

    @abc.abstractmethod
    def clear(self) -> None: ...

    def failure_exception(self) -> None:
        raise RuntimeError(getattr(self, "state", None) and self.state.failure or "KV send failed")


class KVReceiver(abc.ABC):
    """Decode side, one per request."""

    @abc.abstractmethod
    def init(self, dst_pages, transfer_id: str, prefill_addr: str) -> None: ...

    @abc.abstractmethod
    def poll(self) -> KVPoll: ...

    @abc.abstractmethod
    def abort(self) -> None: ...

    @abc.abstractmethod
    def clear(self) -> None: ...

    def failure_exception(self) -> None:
        raise RuntimeError(getattr(self, "state", None) and self.state.failure or "KV receive failed")


class KVManager(abc.ABC):
    """Per-engine factory of senders / receivers."""

    @abc.abstractmethod
    def create_sender(self, req_id: str) -> KVSender: ...

    @abc.abstractmethod
    def create_receiver(self, req_id: str) -> KVReceiver: ...
