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
        from ...models.clip import CLIPTextModel
        classes = {"UMT5EncoderModel": UMT5EncoderModel, "T5EncoderModel": T5EncoderModel}
        names = [c.strip() for c in stage_config.model_class.split(",")]
        subs = [s.strip() for s in (stage_config.stage_sub_dir or "text_encoder").split(",")]
        name = next((c for c in names if c in classes), "UMT5EncoderModel")
        sub = subs[names.index(name)] if name in names and len(subs) == len(names) else subs[-1]
        cfg = load_stage_config(model_dir, sub, config_overrides)
        self.model = load_stage_model(classes[name], cfg, model_dir, sub, self.device, self.dtype, seed=11)
        # a second, pooled prompt encoder (Flux: CLIP beside T5) when the stage lists one and its
        # directory exists; its vector conditions the denoiser's time embedding
        self.pooled_model = None
        if "CLIPTextModel" in names and model_dir and len(subs) == len(names):
            import os
            csub = subs[names.index("CLIPTextModel")]
            if os.path.exists(os.path.join(model_dir, csub, "config.json")):
                ccfg = load_stage_config(model_dir, csub, None)
                self.pooled_model = load_stage_model(CLIPTextModel, ccfg, model_dir, csub, self.device, self.dtype, seed=12)
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
        if self.pooled_model is not None:
            for r in reqs:
                # ids from the pooled encoder's own tokenizer when the front end supplied them
                cids = r.data.get("clip_input_ids") or r.data["input_ids"]
                pc = self.pooled_model.cfg
                t = torch.as_tensor(list(cids)[: pc.max_position_embeddings], dtype=torch.long, device=self.device)
                t = t.clamp_max(pc.vocab_size - 1).view(1, -1)
                r.data["pooled_text_embeds"] = self.pooled_model(t, return_pooled=True)[1][0]
        k = 0
        for r in reqs:
            r.data["text_embeds"] = emb[k]
            k += 1
            if r.data.get("negative_input_ids") is not None:
                r.data["negative_text_embeds"] = emb[k]
                k += 1
