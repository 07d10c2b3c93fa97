from .kv_manager import KVManager, KVPoll, KVReceiver, KVSender, StateHolder  # noqa: F401
