"""Hands GPUs to stages (reference `multimodal/manager/device_manager.py`): stages get disjoint
device lists in stage order when enough GPUs exist, otherwise they share round-robin (or all run
on the CPU when no GPU is present)."""

from __future__ import annotations

import torch


class DeviceManager:
    def __init__(self, num_devices: int | None = None, device_type: str | None = None):
        if device_type is None:
            device_type = "cuda" if torch.cuda.is_available() else "cpu"
        self.device_type = device_type
        self.num_devices = num_devices if num_devices is not None else \
            (torch.cuda.device_count() if device_type == "cuda" else 1)
        self.assigned: dict[int, list[str]] = {}
        self._next = 0

    def allocate(self, stage_id: int, num_gpus: int) -> list[str]:
        if self.device_type == "cpu":
            devs = ["cpu"]
        else:
            devs = []
            for _ in range(max(1, num_gpus)):
                devs.append(f"cuda:{self._next % self.num_devices}")
                self._next += 1
        self.assigned[stage_id] = devs
        return devs

    def oversubscribed(self) -> bool:
        used = [d for ds in self.assigned.values() for d in ds]
        return len(used) != len(set(used))
