"""Quantisation recipe of a run (reference `python/sgl_jax/srt/configs/quantization_config.py`):
which modules are quantised, to what dtype, with which scale granularity, and whether the
checkpoint already is quantised (static) or is quantised while loading (dynamic)."""

from __future__ import annotations

import dataclasses
import os
import re

import torch
import yaml

_DTYPES = {"float8_e4m3fn": torch.float8_e4m3fn, "float8_e5m2": torch.float8_e5m2, "int8": torch.int8,
           "bfloat16": torch.bfloat16, None: None, "null": None}
PRESET_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "utils", "quantization_configs")


@dataclasses.dataclass
class LinearRule:
    module_path: str
    weight_dtype: torch.dtype | None
    activation_dtype: torch.dtype | None = None

    def matches(self, name: str) -> bool:
        return re.fullmatch(self.module_path, name) is not None or re.search(self.module_path, name) is not None


@dataclasses.dataclass
class QuantizationConfig:
    name: str = ""
    is_static_checkpoint: bool = False
    weight_block_size: tuple[int, int] | None = None
    granularity: str = "per_channel"            # per_tensor | per_channel | block
    allow_narrow_n_blockwise: bool = False
    linear_rules: list[LinearRule] = dataclasses.field(default_factory=list)
    moe_weight_dtype: torch.dtype | None = None
    moe_activation_dtype: torch.dtype | None = None
    moe_weight_block_size: tuple[int, int] | None = None

    @classmethod
    def from_yaml(cls, path: str) -> "QuantizationConfig":
        with open(path) as f:
            q = yaml.safe_load(f)["quantization"]
        wbs = tuple(q["weight_block_size"]) if q.get("weight_block_size") else None
        rules = [LinearRule(r["module_path"], _DTYPES[r.get("weight_dtype")], _DTYPES[r.get("activation_dtype")])
                 for r in (q.get("linear") or {}).get("rules", [])]
        moe = q.get("moe") or {}
        return cls(name=os.path.splitext(os.path.basename(path))[0],
                   is_static_checkpoint=bool(q.get("is_static_checkpoint", False)), weight_block_size=wbs,
                   granularity=q.get("granularity") or ("block" if wbs else "per_channel"),
                   allow_narrow_n_blockwise=bool(q.get("allow_narrow_n_blockwise", False)), linear_rules=rules,
                   moe_weight_dtype=_DTYPES[moe.get("weight_dtype")],
                   moe_activation_dtype=_DTYPES[moe.get("activation_dtype")],
                   moe_weight_block_size=tuple(moe["weight_block_size"]) if moe.get("weight_block_size") else wbs)

    @classmethod
    def resolve(cls, quantization: str | None, config_path: str | None = None, hf_config=None) -> "QuantizationConfig | None":
        """`--quantization-config-path` wins; `--quantization <preset>` names a bundled YAML;
        otherwise a `quantization_config` block inside the HF config selects the static FP8 recipe
        (reference `model_config.py:325`)."""
        if config_path:
            return cls.from_yaml(config_path)
        if quantization:
            path = os.path.join(PRESET_DIR, quantization + ".yaml")
            if not os.path.exists(path):
                raise ValueError(f"unknown quantization preset {quantization!r}; available: {sorted(presets())}")
            return cls.from_yaml(path)
        hq = getattr(hf_config, "quantization_config", None) if hf_config is not None else None
        if isinstance(hq, dict) and hq.get("quant_method") == "fp8":
            cfg = cls.from_yaml(os.path.join(PRESET_DIR, "fp8_deepseek_v3.yaml"))
            if hq.get("weight_block_size"):
                cfg.weight_block_size = tuple(hq["weight_block_size"])
                cfg.moe_weight_block_size = cfg.weight_block_size
            return cfg
        return None

    def rule_for(self, module_name: str) -> LinearRule | None:
        for r in self.linear_rules:
            if r.matches(module_name):
                return r if r.weight_dtype is not None else None
        return None


def presets() -> list[str]:
    return [f[:-5] for f in os.listdir(PRESET_DIR) if f.endswith(".yaml")]
