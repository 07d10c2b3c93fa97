"""One adapter's weights on the host, regrouped per layer and fused module."""

from __future__ import annotations

import glob
import os
import re

import torch

from .lora_config import STACK_COUNT, STACKED, LoRAConfig

_LAYER_RE = re.compile(r"layers\.(\d+)\.")


class LoRAAdapter:
    """`weights[layer][fused_module] = (A, B)` with `A = [stack, r, in]`, `B = list of [out_j, r]`
    (missing members of a fusion are zero)."""

    def __init__(self, uid: str, config: LoRAConfig):
        self.uid = uid
        self.config = config
        self.scaling = config.scaling
        self.r = config.r
        self.weights: dict[int, dict[str, tuple[list, list]]] = {}

    @classmethod
    def from_path(cls, uid: str, path: str) -> "LoRAAdapter":
        cfg = LoRAConfig(path)
        ad = cls(uid, cfg)
        tensors: dict[str, torch.Tensor] = {}
        files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
        if files:
            from safetensors.torch import load_file
            for f in files:
                tensors.update(load_file(f))
        else:
            for f in sorted(glob.glob(os.path.join(path, "*.bin")) + glob.glob(os.path.join(path, "*.pt"))):
                tensors.update(torch.load(f, map_location="cpu", weights_only=True))
        if not tensors:
            raise ValueError(f"no adapter weights found in {path}")
        ad.ingest(tensors)
        return ad

    def ingest(self, tensors: dict[str, torch.Tensor]):
        for name, w in tensors.items():
            m = _LAYER_RE.search(name)
            if m is None or ("lora_A" not in name and "lora_B" not in name):
                continue
            layer = int(m.group(1))
            mod = None
            for cand in list(STACKED) + ["o_proj", "down_proj", "qkv_proj", "gate_up_proj"]:
                if f".{cand}." in name:
                    mod = cand
                    break
            if mod is None:
                continue
            fused, idx = STACKED.get(mod, (mod, 0))
            n = STACK_COUNT[fused]
            slot = self.weights.setdefault(layer, {}).setdefault(fused, ([None] * n, [None] * n))
            if mod in ("qkv_proj", "gate_up_proj"):
                # checkpoint already fused: A shared, B covers the whole output
                slot[0 if "lora_A" in name else 1][0] = w
                slot[0 if "lora_A" in name else 1][1:] = ["fused"] * (n - 1)
            else:
                slot[0 if "lora_A" in name else 1][idx] = w
