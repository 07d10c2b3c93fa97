"""The denoising loop (reference `multimodal/manager/scheduler/diffusion_scheduler.py`,
`model_executor/diffusion`): seeded latents, `num_inference_steps` transformer evaluations (two
per step under classifier-free guidance), one solver step each; abort is honoured between steps."""

from __future__ import annotations

import torch

from ...model_executor.loading import load_stage_config, load_stage_model
from ...models.diffusion_solvers import SOLVERS
from .base import StageScheduler


class DiffusionScheduler(StageScheduler):
    name = "diffusion"

    def __init__(self, stage_config, devices, model_dir, dtype=torch.bfloat16, config_overrides=None, **kw):
        super().__init__(stage_config, devices, model_dir, dtype)
        from ...models.dit import WanTransformer3DModel
        from ...models.flux import FluxTransformer2DModel
        self._flux_cls = FluxTransformer2DModel
        classes = {"WanTransformer3DModel": WanTransformer3DModel, "FluxTransformer2DModel": FluxTransformer2DModel}
        sub = stage_config.stage_sub_dir or "transformer"
        cfg = load_stage_config(model_dir, sub, config_overrides)
        self.model = load_stage_model(classes[stage_config.model_class], cfg, model_dir, sub, self.device, self.dtype,
                                      seed=12)
        sp = stage_config.scheduler_params
        self.solver_cls = SOLVERS[sp.get("Scheduler", "FlowMatchEulerDiscreteScheduler")]
        self.shift = float(sp.get("flow_shift", 1.0))
        self.vae_scale = int(sp.get("vae_scale_factor", 8))
        self.vae_temporal = int(sp.get("vae_temporal_factor", 4))
        self.steps_run = 0

    @torch.inference_mode()
    def run_batch(self, reqs):
        for r in reqs:
            d = r.data
            c = self.model.config
            T = (d["num_frames"] - 1) // self.vae_temporal + 1
            H, W = d["height"] // self.vae_scale, d["width"] // self.vae_scale
            pt, ph, pw = self.model.patch
            T, H, W = max(T // pt, 1) * pt, max(H // ph, 1) * ph, max(W // pw, 1) * pw
            g = torch.Generator().manual_seed(int(d["seed"]))
            flux = isinstance(self.model, self._flux_cls)
            if flux:
                T = 1                        # an image model: one frame, latents packed 2x2 inside the model
            x = torch.randn(1, self.model.vae_channels if flux else c.in_channels, T, H, W,
                            generator=g).to(self.device, self.dtype)
            solver = self.solver_cls(shift=self.shift)
            solver.set_timesteps(int(d["num_inference_steps"]), self.device)
            text = d["text_embeds"][None].to(self.device)
            extra = {}
            if flux:
                if d.get("pooled_text_embeds") is not None:
                    extra["pooled"] = d["pooled_text_embeds"][None].to(self.device)
                extra["guidance"] = torch.full((1,), float(d.get("embedded_guidance", 3.5)), device=self.device)
            neg = d.get("negative_text_embeds")
            gs = float(d.get("guidance_scale", 1.0))
            for t in solver.timesteps:
                if self.is_aborted(r):
                    r.aborted = True
                    break
                tt = t.reshape(1).to(self.device)
                v = self.model(x, tt, text, **extra)
                if neg is not None and gs != 1.0:
                    L = max(text.shape[1], neg.shape[0])
                    n = torch.zeros(1, L, neg.shape[-1], dtype=neg.dtype, device=self.device)
                    n[0, :neg.shape[0]] = neg
                    vn = self.model(x, tt, n, **extra)
                    v = vn + gs * (v - vn)
                x = solver.step(v, x)
                self.steps_run += 1
            d["latents"] = x
