"""`/start_profile` handling inside the scheduler.

Reference: `python/sgl_jax/srt/managers/scheduler_profiler_mixing.py` (`_StageBasedTrigger` :26,
`_ProfileManager` :86, `start_profile` :161, batch predicate :321).  The trace itself comes
from `torch.profiler` (CUPTI kernels + CPU ops, chrome-trace JSON) instead of the JAX
profiler; stop is automatic after `num_steps` forward steps, or per stage (prefill /
decode) with `profile_by_stage`.
"""

from __future__ import annotations

import logging
import os
import time

from .io_struct import ProfileReq, ProfileReqOutput, ProfileReqType

logger = logging.getLogger(__name__)


class _StageBasedTrigger:
    """Counts forward steps per stage and tells when a stage's quota is used up."""

    def __init__(self, stages: list[str], num_steps: int):
        self.remaining = {s: num_steps for s in stages}
        self.active: str | None = None

    def step(self, stage: str) -> tuple[bool, bool]:
        """Returns (start_now, stop_now) for a batch of `stage`."""
        start = stop = False
        if self.active is not None and stage != self.active:
            stop = True
            self.active = None
        if stage in self.remaining and self.remaining[stage] > 0:
            if self.active is None:
                start = True
                self.active = stage
            self.remaining[stage] -= 1
            if self.remaining[stage] == 0:
                del self.remaining[stage]
                self._pending_stop = True
        return start, stop

    @property
    def done(self) -> bool:
        return not self.remaining and self.active is None


class SchedulerProfilerMixin:
    def init_profiler(self):
        self.profiler = None
        self.profile_id: str | None = None
        self.profile_output_dir: str | None = None
        self.profile_steps_left: int | None = None
        self.profile_start_step: int | None = None
        self.profile_stage_trigger: _StageBasedTrigger | None = None
        self.profile_in_progress = False

    def profile(self, req: ProfileReq) -> ProfileReqOutput:
        if req.type == ProfileReqType.START_PROFILE:
            return self.start_profile(req)
        if req.type == ProfileReqType.STOP_PROFILE:
            return self.stop_profile()
        return ProfileReqOutput(True, "profiling" if self.profile_in_progress else "idle")

    def start_profile(self, req: ProfileReq) -> ProfileReqOutput:
        if self.profile_in_progress:
            return ProfileReqOutput(False, "Profiling is already in progress. Call /stop_profile first.")
        self.profile_output_dir = req.output_dir or os.environ.get("SGLANG_PROFILER_DIR", "/tmp/sglang_profile")
        os.makedirs(self.profile_output_dir, exist_ok=True)
        self.profile_id = req.profile_id or str(int(time.time()))
        self.profile_steps_left = req.num_steps
        self.profile_start_step = req.start_step
        self.profile_activities = [a.upper() for a in (req.activities or ["CPU", "GPU"])]
        if req.profile_by_stage:
            self.profile_stage_trigger = _StageBasedTrigger(req.profile_stages or ["prefill", "decode"],
                                                            req.num_steps or 5)
            self.profile_in_progress = True
            return ProfileReqOutput(True, "Succeeded (stage based)")
        if req.start_step is None:
            self._begin_trace()
        self.profile_in_progress = True
        return ProfileReqOutput(True, "Succeeded")

    def _begin_trace(self):
        import torch
        want = getattr(self, "profile_activities", None) or ["CPU", "GPU"]
        acts = [torch.profiler.ProfilerActivity.CPU] if "CPU" in want or not torch.cuda.is_available() else []
        if "GPU" in want and torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        mem = "MEM" in want
        if mem and torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=100000)     # allocator history for memory_viz
        self.profiler = torch.profiler.profile(activities=acts or [torch.profiler.ProfilerActivity.CPU],
                                               record_shapes=False, with_stack=False, profile_memory=mem)
        self.profiler.start()

    def _end_trace(self, suffix: str = ""):
        if self.profiler is None:
            return
        self.profiler.stop()
        path = os.path.join(self.profile_output_dir, f"{self.profile_id}{suffix}-TP-{self.tp_rank}.trace.json.gz")
        self.profiler.export_chrome_trace(path)
        logger.info("Profiler trace written to %s", path)
        self.profiler = None
        import torch
        if "MEM" in (getattr(self, "profile_activities", None) or []) and torch.cuda.is_available():
            snap = os.path.join(self.profile_output_dir, f"{self.profile_id}{suffix}-TP-{self.tp_rank}-memory.pickle")
            torch.cuda.memory._dump_snapshot(snap)
            torch.cuda.memory._record_memory_history(enabled=None)
            logger.info("Memory snapshot written to %s", snap)

    def stop_profile(self) -> ProfileReqOutput:
        if not self.profile_in_progress:
            return ProfileReqOutput(False, "Profiling is not in progress. Call /start_profile first.")
        self._end_trace()
        self.profile_in_progress = False
        self.profile_stage_trigger = None
        self.profile_steps_left = None
        return ProfileReqOutput(True, "Succeeded")

    def _profile_batch_predicate(self, batch):
        """Called once per forward step, before launch."""
        if not self.profile_in_progress:
            return
        if self.profile_stage_trigger is not None:
            stage = "prefill" if batch.forward_mode.is_extend() else "decode"
            start, stop = self.profile_stage_trigger.step(stage)
            if stop:
                self._end_trace(f"-{self._profile_stage_name}")
            if start:
                self._profile_stage_name = stage
                self._begin_trace()
            if self.profile_stage_trigger.done:
                self._end_trace(f"-{getattr(self, '_profile_stage_name', 'stage')}")
                self.profile_in_progress = False
                self.profile_stage_trigger = None
            return
        if self.profile_start_step is not None:
            if self.forward_ct >= self.profile_start_step and self.profiler is None:
                self._begin_trace()
                self.profile_start_step = None
            else:
                return
        if self.profile_steps_left is not None:
            self.profile_steps_left -= 1
            if self.profile_steps_left < 0:
                self.stop_profile()
