"""Transfer backend selection by name (reference `python/sgl_jax/srt/disaggregation/factory.py`)."""

from __future__ import annotations


def create_transfer_backend(name: str, device_pool, **kw):
    from .transfer.zmq_transfer import ZmqTransferBackend
    if name in ("tcp", "zmq", "host"):
        return ZmqTransferBackend(device_pool, mode="tcp", **kw)
    if name in ("cuda_ipc", "nvlink"):
        return ZmqTransferBackend(device_pool, mode="cuda_ipc", **kw)
    raise ValueError(f"unknown KV transfer backend {name!r} (tcp | cuda_ipc)")
