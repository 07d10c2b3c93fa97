"""What a stage scheduler provides: `run_batch` mutates the requests' `data` in place."""

from __future__ import annotations

import torch


class StageScheduler:
    name = "base"

    def __init__(self, stage_config, devices, model_dir: str | None, dtype=torch.bfloat16, **kw):
        self.cfg = stage_config
        self.device = torch.device(devices[0])
        self.model_dir = model_dir
        self.dtype = dtype if self.device.type == "cuda" else torch.float32
        self._aborted: set[str] = set()

    def abort(self, rid: str):
        self._aborted.add(rid)

    def is_aborted(self, req) -> bool:
        return req.aborted or req.rid in self._aborted

    def run_batch(self, reqs):
        raise NotImplementedError
