"""The LoRA routing of the forward pass that is currently running.

Layers read it instead of threading an argument through every model's `forward`
(reference `python/sgl_jax/srt/lora/context_manager.py`)."""

from __future__ import annotations

import contextlib

from .backend.base_backend import LoRABatchInfo

_current: LoRABatchInfo | None = None


def current() -> LoRABatchInfo | None:
    return _current


@contextlib.contextmanager
def lora_batch(info: LoRABatchInfo | None):
    global _current
    prev = _current
    _current = info
    try:
        yield
    finally:
        _current = prev
