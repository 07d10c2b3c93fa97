"""`named_scope`: names a region in profiler timelines (reference
`python/sgl_jax/srt/utils/profiling_utils.py:6`, which wraps `jax.named_scope`); here the region is
an NVTX range on a GPU and a no-op otherwise."""

from __future__ import annotations

import contextlib
import functools

import torch


@contextlib.contextmanager
def _range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def named_scope(arg=None, *, name: str | None = None):
    """Usable as `@named_scope`, `@named_scope(name="x")` or `with named_scope("x"):`."""
    if isinstance(arg, str):
        return _range(arg)
    if callable(arg):
        fn = arg
        label = name or getattr(fn, "__qualname__", "scope")

        @functools.wraps(fn)
        def wrapped(*a, **k):
            with _range(label):
                return fn(*a, **k)
        return wrapped

    def deco(fn):
        return named_scope(fn, name=name)
    return deco
