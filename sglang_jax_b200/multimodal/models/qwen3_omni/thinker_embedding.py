"""First stage of the Qwen3-Omni pipeline (reference
`python/sgl_jax/srt/multimodal/models/qwen3_omni_moe/qwen3_omni_thinker_embedding.py`): run the
audio and vision encoders, scatter their outputs over the placeholder tokens of the prompt's
embedding, compute the three-stream rotary positions, and collect the deep-stack features — the
`mm_inputs` the language-model stage consumes."""

from __future__ import annotations

from typing import Iterable

import numpy as np
import torch
from torch import nn

from ...manager.mrope_utils import get_rope_index
from .audio_encoder import Qwen3OmniMoeAudioEncoder, feat_lengths
from .vision_encoder import Qwen3OmniMoeVisionEncoder


def _ns(c):
    from types import SimpleNamespace
    return SimpleNamespace(**c) if isinstance(c, dict) else c


class Qwen3OmniMoeThinkerEmbedding(nn.Module):
    def __init__(self, config, dtype=torch.bfloat16):
        super().__init__()
        thinker = _ns(getattr(config, "thinker_config", None) or config)
        self.config = thinker
        text = _ns(thinker.text_config)
        self.audio_tower = Qwen3OmniMoeAudioEncoder(_ns(thinker.audio_config), dtype)
        self.visual = Qwen3OmniMoeVisionEncoder(_ns(thinker.vision_config), dtype)
        self.embed_tokens = nn.Embedding(text.vocab_size, text.hidden_size, dtype=dtype)
        self.embed_tokens.weight.requires_grad_(False)
        self.image_token_id = thinker.image_token_id
        self.video_token_id = getattr(thinker, "video_token_id", None)
        self.audio_token_id = thinker.audio_token_id
        self.position_id_per_seconds = getattr(thinker, "position_id_per_seconds", 25)

    @torch.inference_mode()
    def forward(self, input_ids, pixel_values=None, image_grid_thw=None, pixel_values_videos=None,
                video_grid_thw=None, input_features=None, feature_lens=None, second_per_grid_ts=None) -> dict:
        dev = self.embed_tokens.weight.device
        ids = torch.as_tensor(input_ids, dtype=torch.long, device=dev)
        emb = self.embed_tokens(ids).clone()
        deep = None

        def scatter(mask, feats, what):
            if int(mask.sum()) != feats.shape[0]:
                raise ValueError(f"{int(mask.sum())} {what} placeholder tokens for {feats.shape[0]} {what} embeddings")
            emb[mask] = feats.to(emb.dtype)

        for px, grid, tok in ((pixel_values, image_grid_thw, self.image_token_id),
                              (pixel_values_videos, video_grid_thw, self.video_token_id)):
            if px is None:
                continue
            grid = torch.as_tensor(grid).view(-1, 3)
            feats, ds = self.visual(torch.as_tensor(px).to(dev), grid, return_deepstack=True)
            mask = ids == tok
            scatter(mask, feats, "vision")
            if ds:
                if deep is None:
                    deep = torch.zeros(len(ds), len(ids), emb.shape[-1], dtype=emb.dtype, device=dev)
                for i, f in enumerate(ds):
                    deep[i, mask] = f.to(emb.dtype)
        if input_features is not None:
            feats = torch.as_tensor(input_features).to(dev)
            lens = torch.as_tensor(feature_lens if feature_lens is not None else [feats.shape[-1]]).view(-1)
            scatter(ids == self.audio_token_id, self.audio_tower(feats, lens), "audio")
        vis = self.config.vision_config
        merge = vis["spatial_merge_size"] if isinstance(vis, dict) else vis.spatial_merge_size
        pos, delta = get_rope_index(ids.tolist(), image_grid_thw, video_grid_thw, image_token_id=self.image_token_id,
                                    video_token_id=self.video_token_id, spatial_merge_size=merge,
                                    tokens_per_second=self.position_id_per_seconds,
                                    second_per_grid_ts=second_per_grid_ts)
        out = {"input_embedding": emb.cpu(), "mrope_positions": pos, "mrope_position_delta": delta}
        if deep is not None:
            out["deepstack"] = deep.cpu()
        return out

    def audio_token_count(self, num_frames: int) -> int:
        return int(feat_lengths(torch.tensor([num_frames])))

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        a, v = [], []
        loaded = set()
        for name, w in weights:
            n = name[len("thinker."):] if name.startswith("thinker.") else name
            if n.startswith("audio_tower."):
                a.append((n, w))
            elif n.startswith("visual."):
                v.append((n, w))
            elif n in ("model.embed_tokens.weight", "model.language_model.embed_tokens.weight"):
                self.embed_tokens.weight.data.copy_(w.to(self.embed_tokens.weight.dtype))
                loaded.add("embed_tokens.weight")
        loaded |= {"audio_tower." + n for n in self.audio_tower.load_weights(a)}
        loaded |= {"visual." + n for n in self.visual.load_weights(v)}
        return loaded


EntryClass = [Qwen3OmniMoeThinkerEmbedding]
