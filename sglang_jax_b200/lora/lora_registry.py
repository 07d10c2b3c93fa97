"""Front-end bookkeeping of LoRA adapters (reference
`python/sgl_jax/srt/lora/lora_registry.py`).

The tokenizer process resolves the adapter *name* a request carries into a stable
`lora_id`, counts in-flight requests per adapter, and lets an unload wait until the
adapter is idle."""

from __future__ import annotations

import asyncio
import dataclasses
import uuid


@dataclasses.dataclass
class LoRARef:
    lora_id: str = dataclasses.field(default_factory=lambda: uuid.uuid4().hex)
    lora_name: str | None = None
    lora_path: str | None = None
    pinned: bool = False

    def __str__(self):
        return f"LoRARef(id={self.lora_id}, name={self.lora_name}, path={self.lora_path})"


class LoRARegistry:
    def __init__(self, lora_paths: list | dict | None = None):
        self._by_name: dict[str, LoRARef] = {}
        self._counters: dict[str, int] = {}
        self._idle: dict[str, asyncio.Event] = {}
        for ref in parse_lora_paths(lora_paths):
            self._register(ref)

    # ------------------------------------------------------------------
    def _register(self, ref: LoRARef):
        if ref.lora_name in self._by_name:
            raise ValueError(f"LoRA adapter {ref.lora_name!r} is already registered")
        self._by_name[ref.lora_name] = ref
        self._counters[ref.lora_id] = 0

    def register(self, ref: LoRARef):
        self._register(ref)

    def unregister(self, lora_name: str) -> str:
        ref = self._by_name.pop(lora_name, None)
        if ref is None:
            raise ValueError(f"LoRA adapter {lora_name!r} is not loaded; loaded: {sorted(self._by_name)}")
        return ref.lora_id

    def get(self, lora_name: str) -> LoRARef | None:
        return self._by_name.get(lora_name)

    def all(self) -> dict[str, LoRARef]:
        return dict(self._by_name)

    @property
    def num_registered(self) -> int:
        return len(self._by_name)

    # ------------------------------------------------------------------
    def acquire(self, lora_name: str | list | None):
        """Name(s) -> id(s); every acquired id must be `release`d when the request ends."""
        if lora_name is None:
            return None
        if isinstance(lora_name, (list, tuple)):
            return [self.acquire(n) for n in lora_name]
        ref = self._by_name.get(lora_name)
        if ref is None:
            raise ValueError(f"LoRA adapter {lora_name!r} is not loaded; loaded adapters: {sorted(self._by_name)}")
        self._counters[ref.lora_id] += 1
        return ref.lora_id

    def release(self, lora_id: str | list | None):
        if lora_id is None:
            return
        if isinstance(lora_id, (list, tuple)):
            for i in lora_id:
                self.release(i)
            return
        if lora_id in self._counters:
            self._counters[lora_id] = max(0, self._counters[lora_id] - 1)
            if self._counters[lora_id] == 0 and lora_id in self._idle:
                self._idle[lora_id].set()

    def in_flight(self, lora_id: str) -> int:
        return self._counters.get(lora_id, 0)

    async def wait_for_unload(self, lora_id: str):
        """Returns once no request uses the adapter any more."""
        if self._counters.get(lora_id, 0) > 0:
            ev = self._idle.setdefault(lora_id, asyncio.Event())
            await ev.wait()
        self._counters.pop(lora_id, None)
        self._idle.pop(lora_id, None)


def _static_id(name: str) -> str:
    """Adapters named at start-up get an id derived from their name, so that every process
    parsing the same `--lora-paths` agrees on it without talking."""
    import hashlib
    return hashlib.sha1(("lora:" + name).encode()).hexdigest()[:32]


def parse_lora_paths(lora_paths) -> list[LoRARef]:
    """`--lora-paths` accepts `name=path`, bare paths (name = path), dicts
    `{"lora_name":..., "lora_path":..., "pinned":...}` or a mapping name -> path."""
    if not lora_paths:
        return []
    refs = []
    if isinstance(lora_paths, dict):
        return [LoRARef(lora_id=_static_id(k), lora_name=k, lora_path=v) for k, v in lora_paths.items()]
    for item in lora_paths:
        if isinstance(item, LoRARef):
            refs.append(item)
        elif isinstance(item, dict):
            refs.append(LoRARef(lora_id=_static_id(item["lora_name"]), lora_name=item["lora_name"],
                                lora_path=item["lora_path"], pinned=bool(item.get("pinned", False))))
        elif "=" in item:
            name, path = item.split("=", 1)
            refs.append(LoRARef(lora_id=_static_id(name), lora_name=name, lora_path=path))
        else:
            refs.append(LoRARef(lora_id=_static_id(item), lora_name=item, lora_path=item))
    return refs
