"""`adapter_config.json` of a PEFT LoRA checkpoint."""

from __future__ import annotations

import json
import os


class LoRAConfig:
    def __init__(self, path: str | None = None, r: int = 0, lora_alpha: float = 0.0,
                 target_modules: list[str] | None = None):
        self.path = path
        self.hf_config: dict = {}
        if path is not None:
            with open(os.path.join(path, "adapter_config.json")) as f:
                self.hf_config = json.load(f)
            r = int(self.hf_config["r"])
            lora_alpha = float(self.hf_config.get("lora_alpha", r))
            target_modules = self.hf_config.get("target_modules") or []
            if isinstance(target_modules, str):
                target_modules = [target_modules]
        self.r = r
        self.lora_alpha = lora_alpha
        self.target_modules = [normalize_module_name(m) for m in (target_modules or [])]
        self.scaling = lora_alpha / r if r else 0.0


# checkpoint module name -> (fused module in this framework, index inside the fusion)
STACKED = {"q_proj": ("qkv_proj", 0), "k_proj": ("qkv_proj", 1), "v_proj": ("qkv_proj", 2),
           "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1)}
STACK_COUNT = {"qkv_proj": 3, "gate_up_proj": 2, "o_proj": 1, "down_proj": 1}
ALL_TARGETS = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


def normalize_module_name(name: str) -> str:
    return name.split(".")[-1]


def fused_targets(target_modules: list[str]) -> list[str]:
    """The fused modules touched by a list of checkpoint module names (`all` = every one)."""
    if any(m in ("all", "all-linear") for m in target_modules):
        target_modules = ALL_TARGETS
    out: list[str] = []
    for m in target_modules:
        f = STACKED.get(m, (m, 0))[0]
        if f in STACK_COUNT and f not in out:
            out.append(f)
    return out
