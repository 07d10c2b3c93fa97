"""Opt-in framework diagnostics (reference `python/sgl_jax/srt/utils/debug_utils.py`): `SGLANG_FRAMEWORK_LOG_LEVEL`
(0 error .. 4 trace) switches on a listing of every parameter with its shard after the model is loaded, and a
decorator that prints the shapes a function sees.  There the listing shows GSPMD shardings; here a parameter is a
plain tensor on one rank, so the listing shows its local shape, dtype, and which slice of the tensor-parallel layout
the owning layer holds."""

from __future__ import annotations

import functools
import os
from enum import IntEnum

import torch


class FrameworkLogLevel(IntEnum):
    ERROR = 0
    WARN = 1
    INFO = 2
    DEBUG = 3
    TRACE = 4


def level() -> FrameworkLogLevel:
    return FrameworkLogLevel(min(max(int(os.environ.get("SGLANG_FRAMEWORK_LOG_LEVEL", "0")), 0), 4))


def parameter_shardings(model: torch.nn.Module) -> list[str]:
    """One line per parameter: name, local shape, dtype, and the owning layer's place in the tensor-parallel layout."""
    owner = {}
    for mod_name, mod in model.named_modules():
        for pname, _ in mod.named_parameters(recurse=False):
            owner[f"{mod_name}.{pname}" if mod_name else pname] = mod
    lines = []
    for name, p in model.named_parameters():
        mod = owner.get(name)
        tp = getattr(mod, "tp_size", 1) or 1
        where = "replicated" if tp == 1 else f"{type(mod).__name__} shard {getattr(mod, 'tp_rank', 0)}/{tp}"
        lines.append(f"{name}: shape={tuple(p.shape)} dtype={str(p.dtype).replace('torch.', '')} "
                     f"device={p.device} {where}")
    return lines


def print_parameter_shardings(model: torch.nn.Module) -> None:
    if level() < FrameworkLogLevel.DEBUG:
        return
    for line in parameter_shardings(model):
        print(line)


def _describe(x) -> str | None:
    if isinstance(x, torch.Tensor):
        return f"{tuple(x.shape)} {str(x.dtype).replace('torch.', '')} {x.device}"
    return None


def log_shapes(name: str):
    """Decorator: at DEBUG and above, print the tensors a call receives and returns."""
    def decorator(fn):
        if level() < FrameworkLogLevel.DEBUG:
            return fn

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            for i, a in enumerate(args):
                d = _describe(a)
                if d:
                    print(f"{name} input[{i}]: {d}")
            out = fn(*args, **kwargs)
            for i, r in enumerate(out if isinstance(out, tuple) else (out,)):
                d = _describe(r)
                if d:
                    print(f"{name} output[{i}]: {d}")
            return out
        return wrapper
    return decorator
