"""Message channels between the front-end, the scheduler and the detokenizer.

Multi-process mode uses ZMQ PUSH/PULL over `ipc://` endpoints with pickled payloads
(reference `python/sgl_jax/srt/utils/common_utils.py:273`); `--enable-single-process`
swaps in in-process queues with the same interface (reference
`python/sgl_jax/srt/managers/communication.py`).
"""

from __future__ import annotations

import queue
from typing import Any


class QueueSender:
    def __init__(self, q: queue.Queue):
        self.q = q

    def send_pyobj(self, obj: Any):
        self.q.put(obj)


class QueueReceiver:
    def __init__(self, q: queue.Queue):
        self.q = q

    def recv_pyobj(self, timeout: float | None = None):
        return self.q.get(timeout=timeout)

    def recv_nowait(self):
        return self.q.get_nowait()


def get_zmq_socket(context, socket_type, endpoint: str, bind: bool):
    import zmq
    sock = context.socket(socket_type)
    if socket_type in (zmq.PUSH,):
        sock.setsockopt(zmq.SNDHWM, 0)
        sock.setsockopt(zmq.SNDBUF, 1 << 26)
    elif socket_type in (zmq.PULL,):
        sock.setsockopt(zmq.RCVHWM, 0)
        sock.setsockopt(zmq.RCVBUF, 1 << 26)
    if bind:
        sock.bind(endpoint)
    else:
        sock.connect(endpoint)
    return sock
