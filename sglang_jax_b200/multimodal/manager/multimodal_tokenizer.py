"""Front end of the multimodal server (reference `multimodal/manager/multimodal_tokenizer.py`):
turns API requests into tokenised stage-0 messages and resolves the futures when the pipeline
answers."""

from __future__ import annotations

import asyncio
import threading

from .io_struct import (GenerateMMReqInput, MMOutput, TokenizedGenerateMMReqInput)


class ByteTokenizer:
    """Fallback when a pipeline directory ships no tokenizer: UTF-8 bytes + 3 (0 pad, 1 eos, 2 unk)."""
    vocab_size = 259

    def encode(self, text: str) -> list[int]:
        return [b + 3 for b in text.encode("utf-8")] + [1]


class MultimodalTokenizer:
    def __init__(self, global_scheduler, tokenizer=None):
        self.gs = global_scheduler
        self.tokenizer = tokenizer or ByteTokenizer()
        self.pending: dict[str, tuple[asyncio.AbstractEventLoop, asyncio.Future]] = {}
        self._lock = threading.Lock()
        global_scheduler.on_output = self._on_output

    def _encode(self, text: str | None) -> list[int] | None:
        if text is None:
            return None
        t = self.tokenizer
        ids = t.encode(text)
        return list(ids.ids) if hasattr(ids, "ids") else list(ids)

    async def generate(self, obj: GenerateMMReqInput) -> MMOutput:
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        with self._lock:
            self.pending[obj.rid] = (loop, fut)
        self.gs.submit(TokenizedGenerateMMReqInput(
            rid=obj.rid, input_ids=self._encode(obj.prompt), negative_input_ids=self._encode(obj.negative_prompt),
            height=obj.height, width=obj.width, num_frames=obj.num_frames,
            num_inference_steps=obj.num_inference_steps, guidance_scale=obj.guidance_scale, seed=obj.seed,
            output_format=obj.output_format))
        return await fut

    def abort(self, rid: str):
        self.gs.abort(rid)

    def _on_output(self, out: MMOutput):
        with self._lock:
            ent = self.pending.pop(out.rid, None)
        if ent is not None:
            loop, fut = ent
            loop.call_soon_threadsafe(lambda: fut.done() or fut.set_result(out))


class MediaPreprocessor:
    """Turns raw media of a chat request into encoder inputs and expands the prompt's placeholder
    tokens (one `image_token_id` / `audio_token_id` per item in the incoming ids) to one token per
    encoder output.  Geometry comes from the model's `config.json` (`vision_config`, `audio_config`,
    token ids) when a model directory is given, else from defaults of the Qwen2-VL family."""

    def __init__(self, model_dir: str | None = None, overrides: dict | None = None):
        import json
        import os
        cfg = {}
        if model_dir and os.path.exists(os.path.join(model_dir, "config.json")):
            with open(os.path.join(model_dir, "config.json")) as f:
                cfg = json.load(f)
        cfg = cfg.get("thinker_config", cfg)
        cfg.update(overrides or {})
        vis = cfg.get("vision_config") or {}
        self.patch = int(vis.get("patch_size", 14))
        self.merge = int(vis.get("spatial_merge_size", 2))
        self.temporal = int(vis.get("temporal_patch_size", 2))
        self.min_pixels = int(cfg.get("min_pixels", 56 * 56))
        self.max_pixels = int(cfg.get("max_pixels", 14 * 14 * 4 * 1280))
        self.image_token_id = int(cfg.get("image_token_id", 151655))
        self.audio_token_id = int(cfg.get("audio_token_id", 151646))
        aud = cfg.get("audio_config") or {}
        self.n_mels = int(aud.get("num_mel_bins", 128))
        self.sample_rate = int(cfg.get("audio_sample_rate", 16000))

    def __call__(self, input_ids: list[int], images=None, audios=None) -> dict:
        import numpy as np
        from .processors import expand_placeholders, frames_to_patches, load_image, log_mel_spectrogram
        out = {"input_ids": list(input_ids)}
        if images:
            px, grids = [], []
            for im in images:
                arr = load_image(im)
                frames = arr[None] if arr.ndim == 3 else arr
                p, g = frames_to_patches(frames, self.patch, self.merge, self.temporal, min_pixels=self.min_pixels,
                                         max_pixels=self.max_pixels)
                px.append(p)
                grids.append(g)
            out["pixel_values"] = np.concatenate(px)
            out["image_grid_thw"] = np.asarray(grids, np.int64)
            counts = [g[0] * g[1] * g[2] // (self.merge ** 2) for g in grids]
            out["input_ids"] = expand_placeholders(out["input_ids"], self.image_token_id, counts)
        if audios:
            from ..models.qwen3_omni.audio_encoder import feat_lengths
            import torch
            feats = [log_mel_spectrogram(np.asarray(a, np.float32), self.sample_rate, n_mels=self.n_mels) for a in audios]
            lens = [f.shape[1] for f in feats]
            out["audio_features"] = torch.cat(feats, dim=1).numpy()
            out["audio_feature_lens"] = np.asarray(lens, np.int64)
            counts = [int(feat_lengths(torch.tensor([n]))) for n in lens]
            out["input_ids"] = expand_placeholders(out["input_ids"], self.audio_token_id, counts)
        return out
