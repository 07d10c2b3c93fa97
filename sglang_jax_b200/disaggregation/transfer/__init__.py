from .zmq_transfer import ZmqTransferBackend  # noqa: F401
