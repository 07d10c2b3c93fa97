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
    """Language backbone over text + audio.

    With a MiMo-Audio backbone (`local_dim` in the model's config, or a `backbone` override) the
    model steps over groups of `group_size` frames: prompt audio becomes speech groups embedded by
    the patch encoder, and every generated `empty` text token triggers the patch decoder, whose
    codes feed the next step.  With a plain language model, first-quantiser codes are mapped into
    the vocabulary above `audio_token_offset` instead."""
    name = "audio_backbone"

    def __init__(self, stage_config, devices, model_dir, dtype=torch.bfloat16, config_overrides=None, **kw):
        super().__init__(stage_config, devices, model_dir, dtype)
        from .vit_scheduler import LLMStageScheduler
        ov = dict(config_overrides or {})
        self.audio_offset = int(ov.pop("audio_token_offset", 0))
        self.codebook = int(ov.pop("codebook_size", 1024))
        self.num_q = int(ov.pop("num_quantizers", 1))
        backbone = ov.pop("backbone", None)
        self.empty_idx = int(ov.pop("empty_idx", 151667))
        self.eos_ids = set(ov.pop("eos_token_ids", []) or [])
        self.llm = LLMStageScheduler(stage_config, devices, model_dir, dtype, ov)
        self.local = None
        hf = self.llm.runner.model_config.hf_config
        if backbone is not None or getattr(hf, "local_dim", None):
            import glob
            import os
            from types import SimpleNamespace
            from ...model_executor.loading import init_dummy
            from ...models.mimo_audio_backbone import MiMoAudioLocalModules
            cfg = SimpleNamespace(**({k: getattr(hf, k) for k in dir(hf) if not k.startswith("_")
                                      and not callable(getattr(hf, k))} | (backbone or {})))
            self.local = MiMoAudioLocalModules(cfg, dtype=self.llm.runner.dtype)
            path = ov.get("model_path") or model_dir
            files = sorted(glob.glob(os.path.join(path, "*.safetensors"))) if path else []
            got = set()
            if files and self.llm.runner.server_args.load_format != "dummy":
                from safetensors.torch import load_file
                for f in files:
                    got |= self.local.load_weights(load_file(f).items())
            if not got:
                init_dummy(self.local, 51)
            self.local.to(self.device).eval()

    @torch.inference_mode()
    def _run_grouped(self, r):
        """MiMo-Audio: one language-model position per group of frames."""
        lm, loc, gen = self.llm.runner, self.local, self.llm.gen
        table = lm.model.get_embed_and_head()[0]
        G, C = loc.group, loc.channels
        text = list(r.data.get("input_ids") or [])
        codes = r.data.get("audio_codes")
        empties = torch.tensor(loc.empty_ids)
        speech = torch.empty(0, G, C, dtype=torch.long)
        if codes is not None:
            codes = torch.as_tensor(codes).long()[:, :C]
            pad = (-codes.shape[0]) % G
            if pad:
                codes = torch.cat([codes, empties[: codes.shape[1]].expand(pad, -1)])
            speech = codes.view(-1, G, codes.shape[1])
            if speech.shape[-1] < C:                         # codec with fewer quantisers than channels
                speech = torch.cat([speech, empties[speech.shape[-1]:].expand(speech.shape[0], G, -1)], dim=-1)
        n_text, n_sp = len(text), speech.shape[0]
        ids = text + [self.empty_idx] * n_sp
        t = torch.tensor(ids, device=table.device)
        emb = table[t.clamp_max(table.shape[0] - 1)] * (t != self.empty_idx)[:, None]
        if n_sp:
            all_sp = torch.cat([empties.expand(n_text, G, C), speech]).to(table.device)
            is_sp = torch.arange(len(ids), device=table.device) >= n_text
            emb = emb + loc.group_embeds(all_sp, is_sp).to(emb.dtype)
        sp = r.data.get("sampling_params") or {}
        max_new = int(sp.get("max_new_tokens", 16))
        temp = float(sp.get("temperature", 0.0))
        g = torch.Generator().manual_seed(int(sp.get("seed", 0)))
        gen.begin(len(ids) + max_new)
        gen.temperature = temp
        force_speech = r.data.get("task") == "tts"
        tok, hidden = gen.extend([min(i, table.shape[0] - 1) for i in ids] or [0], emb, capture_hidden=True)
        out_text, out_codes = [], []
        for _ in range(max_new):
            if force_speech:
                tok = self.empty_idx
            if tok == self.empty_idx:
                grp = loc.patch_decode(hidden[-1:].to(table.dtype), temp, g)           # [1, G, C]
                out_codes.append(grp[0].cpu())
                nxt = loc.group_embeds(grp, torch.ones(1, dtype=torch.bool, device=grp.device)).to(table.dtype)
            else:
                out_text.append(tok)
                if tok in self.eos_ids:
                    break
                nxt = table[tok][None]
            if len(out_text) + len(out_codes) >= max_new:
                break
            tok, hidden = gen.step(min(tok, table.shape[0] - 1), nxt, capture_hidden=True)
        r.data["output_ids"] = out_text
        if out_codes:
            r.data["gen_codes"] = torch.cat(out_codes)

    @torch.inference_mode()
    def run_batch(self, reqs):
        for r in reqs:
            if self.local is not None:
                self._run_grouped(r)
                continue
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
