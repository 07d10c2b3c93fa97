"""Latents -> pixels (reference `multimodal/manager/scheduler/vae_scheduler.py`, `model_executor/vae`)."""

from __future__ import annotations

import torch

from ...model_executor.loading import load_stage_config, load_stage_model
from .base import StageScheduler


class VaeScheduler(StageScheduler):
    name = "vae"

    def __init__(self, stage_config, devices, model_dir, dtype=torch.bfloat16, config_overrides=None, **kw):
        super().__init__(stage_config, devices, model_dir, dtype)
        from ...models.vae import AutoencoderKL, AutoencoderKLWan
        from ...models.wan_vae import WanVAE
        # "AutoencoderKLWan": the reduced causal decoder; "WanVAE": the full encoder / decoder with feature cache
        classes = {"AutoencoderKLWan": AutoencoderKLWan, "AutoencoderKL": AutoencoderKL, "WanVAE": WanVAE}
        sub = stage_config.stage_sub_dir or "vae"
        cfg = load_stage_config(model_dir, sub, config_overrides)
        # decoding in fp32: group norms over large activations lose too much in bf16
        self.model = load_stage_model(classes[stage_config.model_class], cfg, model_dir, sub, self.device,
                                      torch.float32, seed=13)

    @torch.inference_mode()
    def run_batch(self, reqs):
        for r in reqs:
            if r.aborted or "latents" not in r.data:
                continue
            px = self.model.decode(r.data.pop("latents").float())
            # the causal decoder emits `factor` frames per latent frame; the first latent frame stands for
            # one real frame only, so the leading duplicates are dropped
            want = int(r.data.get("num_frames", px.shape[2]))
            if px.shape[2] > want:
                px = px[:, :, -want:]
            r.data["pixels"] = ((px.clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8)[0].cpu()      # [C, T, H, W]
