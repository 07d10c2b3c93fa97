"""Orchestrates the stage pipeline (reference `multimodal/manager/global_scheduler.py`): requests
are dispatched by message type into stage 0, hop from stage to stage through queues, and leave
through the detokenizer callback; an abort reaches the stage that currently holds the request."""

from __future__ import annotations

import dataclasses
import logging
import queue
import threading

from ..configs.stage_config import PipelineConfig
from .device_manager import DeviceManager
from .io_struct import (AbortMMReq, MMOutput, MMReq, TokenizedGenerateAudioReqInput, TokenizedGenerateMMReqInput,
                        TokenizedGenerateOmniReqInput)
from .stage import Stage

logger = logging.getLogger(__name__)


@dataclasses.dataclass
class ReqTrackingState:
    req: MMReq
    current_stage: int = -1


class TypeBasedDispatcher:
    def __init__(self, mapping):
        self._mapping = list(mapping)

    def __call__(self, obj):
        for ty, fn in self._mapping:
            if isinstance(obj, ty):
                return fn(obj)
        raise ValueError(f"no handler for {type(obj).__name__}")


def _build_scheduler(stage_cfg, devices, model_dir, overrides):
    from .scheduler.diffusion_scheduler import DiffusionScheduler
    from .scheduler.text_encoder_scheduler import TextEncoderScheduler
    from .scheduler.vae_scheduler import VaeScheduler
    from .scheduler.vit_scheduler import LLMStageScheduler, VitScheduler
    from .scheduler.audio_scheduler import AudioBackboneScheduler, AudioDecoderScheduler, AudioEncoderScheduler
    from .scheduler.omni_scheduler import AutoRegressiveStageScheduler, EmbeddingStageScheduler
    table = {"text_encoder": TextEncoderScheduler, "encoder": TextEncoderScheduler, "diffusion": DiffusionScheduler,
             "vae": VaeScheduler, "vit": VitScheduler, "llm": LLMStageScheduler, "embed": VitScheduler,
             "audio_encoder": AudioEncoderScheduler, "audio_backbone": AudioBackboneScheduler,
             "audio_decoder": AudioDecoderScheduler, "audio": AudioEncoderScheduler,
             "embedding": EmbeddingStageScheduler, "auto_regressive": AutoRegressiveStageScheduler}
    if stage_cfg.scheduler not in table:
        raise ValueError(f"unknown stage scheduler {stage_cfg.scheduler!r}")
    return table[stage_cfg.scheduler](stage_cfg, devices, model_dir,
                                      config_overrides=(overrides or {}).get(stage_cfg.stage_id))


class GlobalScheduler:
    def __init__(self, pipeline: PipelineConfig, model_dir: str | None = None, device_manager: DeviceManager | None = None,
                 config_overrides: dict | None = None):
        self.pipeline = pipeline
        self.devices = device_manager or DeviceManager()
        self.stages: list[Stage] = []
        for sc in pipeline.stages:
            devs = self.devices.allocate(sc.stage_id, sc.num_gpus)
            self.stages.append(Stage(sc, devs, _build_scheduler(sc, devs, model_dir, config_overrides)))
        self.tracking: dict[str, ReqTrackingState] = {}
        self._lock = threading.Lock()
        self.on_output = lambda out: None
        self._dispatch = TypeBasedDispatcher([
            (TokenizedGenerateMMReqInput, self.convert_request),
            (TokenizedGenerateOmniReqInput, self.convert_omni_request),
            (TokenizedGenerateAudioReqInput, self.convert_audio_request),
            (AbortMMReq, lambda a: self.abort(a.rid)),
        ])
        self._routers = []
        for i, st in enumerate(self.stages):
            st.out_queue = queue.Queue()
            t = threading.Thread(target=self._route, args=(i,), daemon=True, name=f"mm-route-{i}")
            self._routers.append(t)
        self._stop = threading.Event()

    # ------------------------------------------------------------------ lifecycle
    def start(self):
        for st in self.stages:
            st.start()
        for t in self._routers:
            t.start()
        return self

    def shutdown(self):
        self._stop.set()
        for st in self.stages:
            st.stop()

    # ------------------------------------------------------------------ intake
    def submit(self, obj):
        return self._dispatch(obj)

    def _enter(self, req: MMReq):
        with self._lock:
            self.tracking[req.rid] = ReqTrackingState(req, 0)
        self.stages[0].in_queue.put(req)

    def convert_request(self, t: TokenizedGenerateMMReqInput):
        self._enter(MMReq(t.rid, "video" if t.num_frames > 1 else "image", dataclasses.asdict(t)))

    def convert_omni_request(self, t: TokenizedGenerateOmniReqInput):
        self._enter(MMReq(t.rid, "omni", dataclasses.asdict(t) | {"pixel_values": t.pixel_values,
                                                                 "image_grid_thw": t.image_grid_thw,
                                                                 "audio_features": t.audio_features,
                                                                 "audio_feature_lens": t.audio_feature_lens}))

    def convert_audio_request(self, t: TokenizedGenerateAudioReqInput):
        self._enter(MMReq(t.rid, "audio", dataclasses.asdict(t) | {"audio": t.audio}))

    def abort(self, rid: str):
        with self._lock:
            st = self.tracking.get(rid)
        if st is None:
            return False
        st.req.aborted = True
        if 0 <= st.current_stage < len(self.stages):
            self.stages[st.current_stage].abort(rid)
        return True

    # ------------------------------------------------------------------ routing
    def _route(self, i: int):
        src = self.stages[i]
        last = i == len(self.stages) - 1
        while not self._stop.is_set():
            try:
                req = src.out_queue.get(timeout=0.1)
            except queue.Empty:
                continue
            if req.error or req.aborted or last:
                self._finish(req)
                continue
            with self._lock:
                tr = self.tracking.get(req.rid)
                if tr is not None:
                    tr.current_stage = i + 1
            self.stages[i + 1].in_queue.put(req)

    def _finish(self, req: MMReq):
        with self._lock:
            self.tracking.pop(req.rid, None)
        err = req.error or ("aborted" if req.aborted else None)
        result = None if err else {k: req.data.get(k) for k in ("pixels", "output_ids", "text", "waveform")
                                   if req.data.get(k) is not None}
        self.on_output(MMOutput(req.rid, req.kind, result, err,
                                {"stage_times": dict(req.stage_times), "output_format": req.data.get("output_format")}))
