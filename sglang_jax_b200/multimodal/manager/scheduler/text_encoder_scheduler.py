"""Prompt encoders (UMT5 / T5 / CLIP) — reference `multimodal/manager/scheduler/encoder_scheduler.py`,
`model_executor/encoder`."""

from __future__ import annotations

import torch

from ...model_executor.loading import load_stage_config, load_stage_model
from .base import StageScheduler


class TextEncoderScheduler(StageScheduler):
    name = "text_encoder"

    def __init__(self, stage_config, devices, model_dir, dtype=torch.bfloat16, config_overrides=None, **kw):
        super().__init__(stage_config, devices, model_dir, dtype)
        from ....models.umt5 import T5EncoderModel, UMT5EncoderModel
        classes = {"UMT5EncoderModel": UMT5EncoderModel, "T5EncoderModel": T5EncoderModel}
        name = next((c for c in stage_config.model_class.split(",") if c.strip() in classes), "UMT5EncoderModel").strip()
        sub = stage_config.stage_sub_dir.split(",")[-1] or "text_encoder"
        cfg = load_stage_config(model_dir, sub, config_overrides)
        self.model = load_stage_model(classes[name], cfg, model_dir, sub, self.device, self.dtype, seed=11)
        self.max_length = int(stage_config.scheduler_params.get("max_length", 512))

    @torch.inference_mode()
    def run_batch(self, reqs):
        seqs = []
        for r in reqs:
            seqs.append(r.data["input_ids"][: self.max_length])
            if r.data.get("negative_input_ids") is not None:
                seqs.append(r.data["negative_input_ids"][: self.max_length])
        L = max(len(s) for s in seqs)
        ids = torch.zeros(len(seqs), L, dtype=torch.long)
        mask = torch.zeros(len(seqs), L, dtype=torch.long)
        for i, s in enumerate(seqs):
            ids[i, :len(s)] = torch.tensor(s)
            mask[i, :len(s)] = 1
        emb = self.model.encode(ids.to(self.device), mask.to(self.device))
        emb = emb * mask.to(self.device)[..., None].to(emb.dtype)          # padded positions carry zeros
        k = 0
        for r in reqs:
            r.data["text_embeds"] = emb[k]
            k += 1
            if r.data.get("negative_input_ids") is not None:
                r.data["negative_text_embeds"] = emb[k]
                k += 1
