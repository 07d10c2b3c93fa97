"""Stages of the omni (audio + vision + text understanding) pipeline (reference
`multimodal/manager/scheduler/embed_scheduler.py` and the `auto_regressive` stage): `embedding`
turns a request's media into per-token language-model inputs; `auto_regressive` hosts a full
serving engine (continuous batching, paged KV, chunked prefill) that generates from them."""

from __future__ import annotations

import glob
import json
import os
from types import SimpleNamespace

import torch

from ...model_executor.loading import init_dummy
from .base import StageScheduler


def _load_config(model_dir, overrides):
    cfg = {}
    if model_dir and os.path.exists(os.path.join(model_dir, "config.json")):
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
    cfg.update(overrides or {})
    return SimpleNamespace(**cfg)


class EmbeddingStageScheduler(StageScheduler):
    name = "embedding"

    def __init__(self, stage_config, devices, model_dir, dtype=torch.bfloat16, config_overrides=None, **kw):
        super().__init__(stage_config, devices, model_dir, dtype)
        from ...models.qwen3_omni.thinker_embedding import Qwen3OmniMoeThinkerEmbedding
        self.model = Qwen3OmniMoeThinkerEmbedding(_load_config(model_dir, config_overrides), dtype=self.dtype)
        files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))) if model_dir else []
        if files:
            from safetensors.torch import load_file

            def it():
                for f in files:
                    yield from load_file(f).items()
            self.model.load_weights(it())
        else:
            init_dummy(self.model, 41)
        self.model.to(self.device).eval()

    @torch.inference_mode()
    def run_batch(self, reqs):
        for r in reqs:
            d = r.data
            d["mm_inputs"] = self.model(d["input_ids"], d.get("pixel_values"), d.get("image_grid_thw"),
                                        d.get("pixel_values_videos"), d.get("video_grid_thw"),
                                        d.get("audio_features"), d.get("audio_feature_lens"))
            for k in ("pixel_values", "pixel_values_videos", "audio_features"):
                d.pop(k, None)


class AutoRegressiveStageScheduler(StageScheduler):
    name = "auto_regressive"

    def __init__(self, stage_config, devices, model_dir, dtype=torch.bfloat16, config_overrides=None, **kw):
        super().__init__(stage_config, devices, model_dir, dtype)
        from ....entrypoints.engine import Engine
        ov = dict(config_overrides or {})
        cpu = self.device.type == "cpu"
        args = dict(model_path=ov.pop("model_path", None) or model_dir, device=self.device.type,
                    dtype="float32" if cpu else "bfloat16", skip_tokenizer_init=True, enable_single_process=True,
                    disable_radix_cache=True, tp_size=max(1, len(devices)) if not cpu else 1,
                    max_running_requests=int(stage_config.max_batch_size or 8))
        args.update(ov)
        self.engine = Engine(**args)

    def run_batch(self, reqs):
        live = [r for r in reqs if not self.is_aborted(r)]
        if not live:
            return
        sps = []
        for r in live:
            sp = dict(r.data.get("sampling_params") or {})
            sp.setdefault("max_new_tokens", 16)
            sp.setdefault("temperature", 0.0)
            sps.append(sp)
        outs = self.engine.generate(input_ids=[list(r.data["input_ids"]) for r in live], sampling_params=sps,
                                    mm_inputs=[r.data.get("mm_inputs") for r in live])
        for r, o in zip(live, outs):
            r.data["output_ids"] = o["output_ids"]
            r.data.pop("mm_inputs", None)

    def shutdown(self):
        self.engine.shutdown()
