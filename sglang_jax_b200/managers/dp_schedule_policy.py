"""Request -> data-parallel rank routing (reference `python/sgl_jax/srt/managers/dp_schedule_policy.py`,
`dp_rank_assignment.py`, `scheduler.py:722-1062`): `round_robin`, `min_running_queue`,
`cache_aware` (longest cached prefix wins, load breaks ties / guards imbalance) and `shape_aware`
(balance prefill tokens)."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class DPRankLoad:
    running: int = 0
    queued: int = 0
    queued_tokens: int = 0
    used_tokens: int = 0


class DPSchedulePolicy:
    name = "base"

    def __init__(self, dp_size: int):
        self.dp_size = dp_size

    def select(self, req, loads: list[DPRankLoad], tree_cache=None) -> int:
        raise NotImplementedError


class RoundRobinPolicy(DPSchedulePolicy):
    name = "round_robin"

    def __init__(self, dp_size):
        super().__init__(dp_size)
        self._next = 0

    def select(self, req, loads, tree_cache=None):
        r = self._next
        self._next = (self._next + 1) % self.dp_size
        return r


class MinRunningQueuePolicy(DPSchedulePolicy):
    name = "min_running_queue"

    def select(self, req, loads, tree_cache=None):
        return min(range(self.dp_size), key=lambda r: (loads[r].running + loads[r].queued, r))


class CacheAwarePolicy(DPSchedulePolicy):
    """Send the request where most of its prompt is already cached, unless that rank is much more
    loaded than the lightest one."""
    name = "cache_aware"

    def __init__(self, dp_size, balance_abs_threshold: int = 32, balance_rel_threshold: float = 1.5,
                 min_match_tokens: int = 16):
        super().__init__(dp_size)
        self.abs_thr, self.rel_thr, self.min_match = balance_abs_threshold, balance_rel_threshold, min_match_tokens

    def select(self, req, loads, tree_cache=None):
        load = [l.running + l.queued for l in loads]
        lightest = min(range(self.dp_size), key=lambda r: (load[r], r))
        if tree_cache is None or getattr(tree_cache, "disable", True):
            return lightest
        from ..mem_cache.radix_cache import RadixKey
        ids = req.origin_input_ids[:-1]
        match = [len(tree_cache.match_prefix(RadixKey(ids, req.extra_key, r)).device_indices)
                 for r in range(self.dp_size)]
        best = max(range(self.dp_size), key=lambda r: (match[r], -load[r], -r))
        if match[best] < self.min_match:
            return lightest
        imbalanced = load[best] - load[lightest] > self.abs_thr and load[best] > self.rel_thr * max(load[lightest], 1)
        return lightest if imbalanced else best


class ShapeAwarePolicy(DPSchedulePolicy):
    """Balance the *prefill tokens* waiting on each rank (long prompts dominate step time)."""
    name = "shape_aware"

    def select(self, req, loads, tree_cache=None):
        return min(range(self.dp_size), key=lambda r: (loads[r].queued_tokens + loads[r].used_tokens // 8,
                                                       loads[r].running + loads[r].queued, r))


_POLICIES = {c.name: c for c in (RoundRobinPolicy, MinRunningQueuePolicy, CacheAwarePolicy, ShapeAwarePolicy)}


def create_dp_schedule_policy(name: str, dp_size: int) -> DPSchedulePolicy:
    if name not in _POLICIES:
        raise ValueError(f"unknown dp_schedule_policy {name}; choose from {sorted(_POLICIES)}")
    return _POLICIES[name](dp_size)


@dataclass
class DPRankAssignment:
    """Sticky request -> rank table (a request keeps its rank across retraction / chunks)."""
    dp_size: int
    table: dict[str, int] = field(default_factory=dict)

    def assign(self, rid: str, rank: int) -> int:
        return self.table.setdefault(rid, rank)

    def get(self, rid: str) -> int | None:
        return self.table.get(rid)

    def release(self, rid: str):
        self.table.pop(rid, None)

    def counts(self) -> list[int]:
        c = [0] * self.dp_size
        for r in self.table.values():
            c[r] += 1
        return c
