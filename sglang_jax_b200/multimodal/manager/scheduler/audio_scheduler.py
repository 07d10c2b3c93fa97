"""Speech pipeline stages (reference `multimodal/manager/scheduler/{audio,audio_backbone}_scheduler.py`):
`audio_encoder` turns a waveform into codec tokens, `audio_backbone` runs the language model over
text + audio tokens, `audio_decoder` turns generated codec tokens back into a waveform."""

from __future__ import annotations

import torch

from ...model_executor.loading import load_stage_config, load_stage_model
from .base import StageScheduler


class _CodecStage(StageScheduler):
    def __init__(self, stage_config, devices, model_dir, dtype=torch.bfloat16, config_overrides=None, **kw):
        super().__init__(stage_config, devices, model_dir, dtype)
        from ...models.audio_codec import MiMoAudioTokenizer
        cfg = load_stage_config(stage_config.model_path if stage_config.model_path and model_dir is None else model_dir,
                                stage_config.stage_sub_dir or "audio_tokenizer", config_overrides)
        self.model = load_stage_model(MiMoAudioTokenizer, cfg, model_dir, stage_config.stage_sub_dir or "audio_tokenizer",
                                      self.device, torch.float32, seed=31)


class AudioEncoderScheduler(_CodecStage):
    name = "audio_encoder"

    @torch.inference_mode()
    def run_batch(self, reqs):
        for r in reqs:
            wave = r.data.get("audio")
            if wave is not None:
                r.data["audio_codes"] = self.model.encode(torch.as_tensor(wave, dtype=torch.float32)).cpu()


class AudioBackboneScheduler(StageScheduler):
    """Language backbone over text + audio tokens: audio codes of the first quantiser are mapped
    into the vocabulary above `audio_token_offset`; for TTS the generated ids are mapped back."""
    name = "audio_backbone"

    def __init__(self, stage_config, devices, model_dir, dtype=torch.bfloat16, config_overrides=None, **kw):
        super().__init__(stage_config, devices, model_dir, dtype)
        from .vit_scheduler import LLMStageScheduler
        ov = dict(config_overrides or {})
        self.audio_offset = int(ov.pop("audio_token_offset", 0))
        self.codebook = int(ov.pop("codebook_size", 1024))
        self.num_q = int(ov.pop("num_quantizers", 1))
        self.llm = LLMStageScheduler(stage_config, devices, model_dir, dtype, ov)

    @torch.inference_mode()
    def run_batch(self, reqs):
        for r in reqs:
            ids = list(r.data.get("input_ids") or [])
            codes = r.data.get("audio_codes")
            if codes is not None:
                ids += (codes[:, 0] + self.audio_offset).tolist()
            sp = r.data.get("sampling_params") or {}
            out = self.llm.gen.generate(ids or [0], None, int(sp.get("max_new_tokens", 16)), float(sp.get("temperature", 0.0)))
            r.data["output_ids"] = out
            if r.data.get("task") == "tts":
                c = torch.tensor([(t - self.audio_offset) % self.codebook for t in out])
                r.data["gen_codes"] = c[:, None].repeat(1, self.num_q)


class AudioDecoderScheduler(_CodecStage):
    name = "audio_decoder"

    @torch.inference_mode()
    def run_batch(self, reqs):
        for r in reqs:
            codes = r.data.get("gen_codes")
            if codes is not None:
                r.data["waveform"] = self.model.decode(codes).cpu()
