"""Vision encoder stage and the language-model stage that consumes its output (reference
`multimodal/manager/scheduler/{vit,embed}_scheduler.py`, `model_executor/vit`)."""

from __future__ import annotations

import torch

from ...model_executor.loading import load_stage_config, load_stage_model
from .base import StageScheduler


class VitScheduler(StageScheduler):
    name = "vit"

    def __init__(self, stage_config, devices, model_dir, dtype=torch.bfloat16, config_overrides=None, **kw):
        super().__init__(stage_config, devices, model_dir, dtype)
        from ...models.qwen2_5_vl_vit import Qwen2_5_VisionTransformer
        sub = stage_config.stage_sub_dir or "visual"
        cfg = load_stage_config(model_dir, sub, config_overrides)
        self.model = load_stage_model(Qwen2_5_VisionTransformer, cfg, model_dir, sub, self.device, self.dtype, seed=21)

    @torch.inference_mode()
    def run_batch(self, reqs):
        # all images of the batch go through the encoder as one packed sequence
        px = [r.data["pixel_values"] for r in reqs if r.data.get("pixel_values") is not None]
        if not px:
            return
        grids = [torch.as_tensor(r.data["image_grid_thw"]).view(-1, 3) for r in reqs if r.data.get("pixel_values") is not None]
        emb = self.model(torch.cat([torch.as_tensor(p) for p in px]), torch.cat(grids))
        off = 0
        unit = self.model.unit
        for r, g in zip([r for r in reqs if r.data.get("pixel_values") is not None], grids):
            n = int((g[:, 0] * g[:, 1] * g[:, 2]).sum()) // unit
            r.data["image_embeds"] = emb[off:off + n]
            off += n
            r.data.pop("pixel_values")


class LLMStageScheduler(StageScheduler):
    """Language backbone of a vision-language pipeline: image embeddings replace the embeddings of
    the `image_token_id` placeholders, then the request is generated like text."""
    name = "llm"

    def __init__(self, stage_config, devices, model_dir, dtype=torch.bfloat16, config_overrides=None, **kw):
        super().__init__(stage_config, devices, model_dir, dtype)
        from ....configs.model_config import ModelConfig
        from ....model_executor.model_runner import ModelRunner
        from ....parallel import state as ps
        from ....server_args import ServerArgs
        ov = dict(config_overrides or {})
        self.image_token_id = int(ov.pop("image_token_id", 151655))
        self.spatial_merge_size = int(ov.pop("spatial_merge_size", 2))
        path = ov.pop("model_path", None) or model_dir
        if not ps.get_state().initialized:
            ps.init_distributed(0, 1, str(self.device))
        sa = ServerArgs(model_path=path, device=self.device.type, dtype="float32" if self.device.type == "cpu" else "bfloat16",
                        page_size=16, skip_tokenizer_init=True, disable_cuda_graph=True, disable_overlap_schedule=True,
                        max_total_tokens=int(ov.pop("max_total_tokens", 4096)), max_running_requests=4,
                        load_format=ov.pop("load_format", "auto"))
        self.runner = ModelRunner(ModelConfig.from_server_args(sa), sa, self.device)
        from ...model_executor.llm_runner import EmbedsGenerator
        self.gen = EmbedsGenerator(self.runner)
        # a language model with multimodal rotary embeddings wants 3-D positions for image tokens
        self.uses_mrope = any(hasattr(m, "mrope_section") for m in self.runner.model.modules())

    @torch.inference_mode()
    def run_batch(self, reqs):
        embed = self.runner.model.get_embed_and_head()[0]
        for r in reqs:
            ids = list(r.data["input_ids"])
            x = None
            img = r.data.get("image_embeds")
            if img is not None:
                t = torch.tensor(ids, device=embed.device)
                x = embed[t.clamp_max(embed.shape[0] - 1)].clone()
                where = (t == self.image_token_id).nonzero().flatten()
                if where.numel() != img.shape[0]:
                    raise ValueError(f"{where.numel()} image placeholder tokens for {img.shape[0]} image embeddings")
                x[where] = img.to(x.dtype).to(x.device)
            sp = r.data.get("sampling_params") or {}
            mpos, delta = None, 0
            if img is not None and self.uses_mrope and r.data.get("image_grid_thw") is not None:
                from ..mrope_utils import get_rope_index
                mpos, delta = get_rope_index(ids, image_grid_thw=r.data["image_grid_thw"],
                                             image_token_id=self.image_token_id,
                                             spatial_merge_size=self.spatial_merge_size)
            r.data["output_ids"] = self.gen.generate(ids, x, int(sp.get("max_new_tokens", 16)),
                                                     float(sp.get("temperature", 0.0)), mrope_positions=mpos,
                                                     mrope_delta=delta)
