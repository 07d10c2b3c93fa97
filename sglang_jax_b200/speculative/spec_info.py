"""Algorithm names and the worker factory (reference
`python/sgl_jax/srt/speculative/spec_info.py`)."""

from __future__ import annotations

from enum import IntEnum, auto


class SpeculativeAlgorithm(IntEnum):
    NONE = auto()
    EAGLE = auto()
    EAGLE3 = auto()
    NEXTN = auto()
    STANDALONE = auto()
    DFLASH = auto()

    @classmethod
    def from_string(cls, name: str | None) -> "SpeculativeAlgorithm":
        if name is None:
            return cls.NONE
        try:
            return cls[name.upper()]
        except KeyError as e:
            raise ValueError(f"unknown speculative algorithm {name!r}") from e

    def is_none(self) -> bool:
        return self == SpeculativeAlgorithm.NONE

    def is_eagle(self) -> bool:
        """Algorithms whose draft consumes target hidden states (bigram radix keys)."""
        return self in (SpeculativeAlgorithm.EAGLE, SpeculativeAlgorithm.EAGLE3, SpeculativeAlgorithm.NEXTN)

    def is_eagle3(self) -> bool:
        return self == SpeculativeAlgorithm.EAGLE3

    def is_nextn(self) -> bool:
        return self == SpeculativeAlgorithm.NEXTN

    def is_standalone(self) -> bool:
        return self == SpeculativeAlgorithm.STANDALONE

    def is_dflash(self) -> bool:
        return self == SpeculativeAlgorithm.DFLASH


def create_spec_worker(server_args, target_worker):
    """Build the worker that wraps `target_worker` for `server_args.speculative_algorithm`."""
    algo = SpeculativeAlgorithm.from_string(server_args.speculative_algorithm)
    if algo.is_none():
        return None
    if algo.is_dflash():
        from .dflash_worker import DFlashWorker
        return DFlashWorker(server_args, target_worker)
    from .eagle_worker import EAGLEWorker
    return EAGLEWorker(server_args, target_worker, algo)
