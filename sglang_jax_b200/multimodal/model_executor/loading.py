"""Builds a stage model from a diffusers/transformers-style sub-directory (`config.json` +
safetensors); with `load_format="dummy"` (or no weights on disk) the weights are seeded noise."""

from __future__ import annotations

import glob
import json
import os
from types import SimpleNamespace

import torch


def load_stage_config(model_dir: str | None, sub_dir: str, overrides: dict | None = None) -> SimpleNamespace:
    cfg = {}
    if model_dir:
        p = os.path.join(model_dir, sub_dir, "config.json")
        if os.path.exists(p):
            with open(p) as f:
                cfg = json.load(f)
    cfg.update(overrides or {})
    return SimpleNamespace(**cfg)


def init_dummy(model: torch.nn.Module, seed: int = 0, std: float = 0.02):
    g = torch.Generator().manual_seed(seed)
    for name, p in model.named_parameters():
        if p.dim() >= 2:
            p.data.copy_(torch.empty(p.shape, dtype=torch.float32).normal_(0, std, generator=g).to(p.dtype))
    return model


def load_stage_model(cls, config, model_dir: str | None, sub_dir: str, device, dtype, seed: int = 0):
    model = cls(config, dtype=dtype)
    files = sorted(glob.glob(os.path.join(model_dir, sub_dir, "*.safetensors"))) if model_dir else []
    if files:
        from safetensors.torch import load_file

        def it():
            for f in files:
                yield from load_file(f).items()
        model.load_weights(it())
    else:
        init_dummy(model, seed)
    return model.to(device).eval()
