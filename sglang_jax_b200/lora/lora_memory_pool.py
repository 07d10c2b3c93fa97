"""Stacked device buffers holding the adapters that can take part in a batch.

Reference: `python/sgl_jax/srt/lora/lora_memory_pool.py` (buffers `[slots, layers, r, dim]`).
Here every (layer, fused module) has `A [slots, stack*r_max, in_local]` and one
`B_j [slots, out_local_j, r_max]` per member of the fusion, already cut to this tensor
rank's shard: column-parallel modules shard B along the output, row-parallel modules shard A
along the input.  Slot assignment is LRU or FIFO over `max_loras_per_batch` slots.
"""

from __future__ import annotations

import logging
from collections import OrderedDict

import torch

from .lora import LoRAAdapter
from .lora_config import STACK_COUNT

logger = logging.getLogger(__name__)


class LoRAMemoryPool:
    def __init__(self, num_slots: int, max_rank: int, dtype, device, eviction_policy: str = "lru"):
        self.num_slots = num_slots
        self.max_rank = max_rank
        self.dtype = dtype
        self.device = device
        self.policy = eviction_policy
        # (layer, module) -> (A, [B_j], shard description)
        self.buffers: dict[tuple[int, str], tuple[torch.Tensor, list[torch.Tensor], dict]] = {}
        self.slot_of: "OrderedDict[str, int]" = OrderedDict()      # uid -> slot, in use order
        self.free_slots = list(range(num_slots))
        self.scalings = torch.zeros(num_slots, dtype=torch.float32, device=device)
        self.ranks = torch.zeros(num_slots, dtype=torch.int32, device=device)

    # ------------------------------------------------------------------ layout
    def add_module(self, layer: int, module: str, linear, shard: dict):
        """`shard` describes how checkpoint tensors map to this rank:
        `{"kind": "column"|"row", "out_slices": [(start, len)] per member, "in_slice": (start, len)}`."""
        stack = STACK_COUNT[module]
        r = self.max_rank
        in_local = shard["in_slice"][1]
        a = torch.zeros(self.num_slots, stack * r, in_local, dtype=self.dtype, device=self.device)
        bs = [torch.zeros(self.num_slots, n, r, dtype=self.dtype, device=self.device) for _, n in shard["out_slices"]]
        self.buffers[(layer, module)] = (a, bs, shard)
        return a, bs

    def get_buffer_bytes(self) -> int:
        n = 0
        for a, bs, _ in self.buffers.values():
            n += a.numel() * a.element_size() + sum(b.numel() * b.element_size() for b in bs)
        return n

    # ------------------------------------------------------------------ slots
    def prepare(self, uids: set[str], adapters: dict[str, LoRAAdapter]) -> dict[str, int]:
        """Make sure every adapter of `uids` sits in a slot; returns uid -> slot."""
        if len(uids) > self.num_slots:
            raise ValueError(f"a batch uses {len(uids)} adapters; --max-loras-per-batch is {self.num_slots}")
        for uid in uids:
            if uid in self.slot_of:
                if self.policy == "lru":
                    self.slot_of.move_to_end(uid)
                continue
            if not self.free_slots:
                victim = next(u for u in self.slot_of if u not in uids)
                self.free_slots.append(self.slot_of.pop(victim))
            slot = self.free_slots.pop(0)
            self._load(adapters[uid], slot)
            self.slot_of[uid] = slot
        return {u: self.slot_of[u] for u in uids}

    def evict(self, uid: str):
        slot = self.slot_of.pop(uid, None)
        if slot is not None:
            self.free_slots.append(slot)

    def _load(self, ad: LoRAAdapter, slot: int):
        if ad.r > self.max_rank:
            raise ValueError(f"adapter rank {ad.r} exceeds --max-lora-rank {self.max_rank}")
        r = ad.r
        for (layer, module), (a_buf, b_bufs, shard) in self.buffers.items():
            a_buf[slot].zero_()
            for b in b_bufs:
                b[slot].zero_()
            w = ad.weights.get(layer, {}).get(module)
            if w is None:
                continue
            a_list, b_list = w
            i0, il = shard["in_slice"]
            fused_ckpt = len(a_list) > 1 and any(isinstance(t, str) for t in a_list[1:])
            for j, (o0, ol) in enumerate(shard["out_slices"]):
                a = a_list[0] if fused_ckpt else a_list[j]
                b = b_list[0] if fused_ckpt else b_list[j]
                if a is None or b is None:
                    continue
                a_buf[slot, j * self.max_rank: j * self.max_rank + r] = a[:, i0:i0 + il].to(self.dtype)
                if fused_ckpt:
                    o0 = shard["fused_out_starts"][j]
                b_bufs[j][slot, :, :r] = b[o0:o0 + ol].to(self.dtype)
        self.scalings[slot] = ad.scaling
        self.ranks[slot] = r
