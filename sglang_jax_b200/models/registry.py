"""Architecture name -> model class (reference `python/sgl_jax/srt/models/registry.py`).
Every module under `models/` exposes `EntryClass` (a class or a list of classes); the
class name is the HF `architectures[0]` string."""

from __future__ import annotations

import importlib
import pkgutil

_REGISTRY: dict[str, type] | None = None


def _scan() -> dict[str, type]:
    from .. import models as pkg
    reg: dict[str, type] = {}
    for m in pkgutil.iter_modules(pkg.__path__):
        if m.name in ("registry",):
            continue
        mod = importlib.import_module(f"{pkg.__name__}.{m.name}")
        entry = getattr(mod, "EntryClass", None)
        if entry is None:
            continue
        for cls in entry if isinstance(entry, (list, tuple)) else [entry]:
            reg[cls.__name__] = cls
    return reg


def get_model_class(architectures: list[str]) -> type:
    global _REGISTRY
    if _REGISTRY is None:
        _REGISTRY = _scan()
    for a in architectures:
        if a in _REGISTRY:
            return _REGISTRY[a]
    raise ValueError(f"Model architectures {architectures} are not supported. "
                     f"Supported: {sorted(_REGISTRY)}")


def supported_architectures() -> list[str]:
    global _REGISTRY
    if _REGISTRY is None:
        _REGISTRY = _scan()
    return sorted(_REGISTRY)
