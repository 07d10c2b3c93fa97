"""Per-module parameter dtypes (`--dtype-config`, reference `python/sgl_jax/srt/configs/dtype_config.py`).

A nested mapping mirrors the module tree, e.g.

    {"default": "bfloat16",
     "model": {"embed_tokens": "float32", "norm": "float32",
               "layers": {"input_layernorm": "float32", "self_attn": {"q_proj": "bfloat16"},
                          "mlp": {"down_proj": "float32"}}},
     "lm_head": "float32"}

A key that is missing falls back to the level's default (the model dtype at the top).  The reference threads the
object through the constructors of one model family; here it is applied to any loaded model by parameter path: layer
indices are skipped, a fused projection takes the entry of its first member (`qkv_proj` <- `q_proj`,
`gate_up_proj` <- `gate_proj`), and only norm weights, embedding tables and plain (unquantised) linear weights are
converted.  A layer whose weight dtype differs from its activations computes in the weight's dtype and hands back
the activation dtype (`ops.linear`, `ops.rmsnorm`), so such layers leave the sm_100a GEMM path.
"""

from __future__ import annotations

import json
from typing import Any

import torch

STR_TO_DTYPE = {"half": torch.float16, "float16": torch.float16, "float": torch.float32, "float32": torch.float32,
                "bfloat16": torch.bfloat16, "int8": torch.int8}
_FUSED_FIRST_MEMBER = {"qkv_proj": "q_proj", "gate_up_proj": "gate_proj"}


def _to_dtype(v) -> torch.dtype:
    if isinstance(v, torch.dtype):
        return v
    if isinstance(v, str) and v.lower() in STR_TO_DTYPE:
        return STR_TO_DTYPE[v.lower()]
    raise ValueError(f"dtype config: {v!r} ({type(v).__name__}) does not name a dtype; known: {sorted(STR_TO_DTYPE)}")


class DtypeConfig:
    def __init__(self, config_dict: dict[str, Any] | None = None, default_dtype=None):
        if config_dict is None and default_dtype is None:
            raise ValueError("a dtype config needs a mapping, a default dtype, or both")
        self.config_dict = self._parse(config_dict or {})
        self.default_dtype = self.config_dict["default"] if "default" in self.config_dict else \
            (_to_dtype(default_dtype) if default_dtype is not None else None)

    def __repr__(self) -> str:
        return f"DtypeConfig(config_dict={self.config_dict!r}, default_dtype={self.default_dtype!r})"

    def _parse(self, d: dict) -> dict:
        return {k: self._parse(v) if isinstance(v, dict) else _to_dtype(v) for k, v in d.items()}

    @classmethod
    def from_arg(cls, arg, default_dtype) -> "DtypeConfig | None":
        """`--dtype-config`: a JSON object, or the path of a file holding one."""
        if not arg:
            return None
        if isinstance(arg, str):
            if arg.lstrip().startswith("{"):
                arg = json.loads(arg)
            else:
                with open(arg, encoding="utf-8") as f:
                    arg = json.load(f)
        return cls(arg, default_dtype)

    def get_config(self, key: str) -> "DtypeConfig":
        sub = self.config_dict.get(key, {})
        return DtypeConfig(sub if isinstance(sub, dict) else {}, self.default_dtype)

    def get_dtype(self, key: str):
        v = self.config_dict.get(key, self.default_dtype)
        return self.default_dtype if isinstance(v, dict) else v

    def get_optional_dtype(self, key: str):
        v = self.config_dict.get(key)
        return None if isinstance(v, dict) else v

    def resolve(self, param_name: str):
        """Dtype of the parameter `model.layers.3.self_attn.qkv_proj.weight`-style path."""
        parts = [p for p in param_name.split(".") if not p.isdigit()]
        if parts and parts[-1] in ("weight", "bias", "scale"):
            parts = parts[:-1]
        if not parts:
            return self.default_dtype
        cfg = self
        for p in parts[:-1]:
            cfg = cfg.get_config(p)
        leaf = parts[-1]
        if leaf not in cfg.config_dict and leaf in _FUSED_FIRST_MEMBER:
            leaf = _FUSED_FIRST_MEMBER[leaf]
        return cfg.get_dtype(leaf)


def apply_dtype_config(model: torch.nn.Module, cfg: DtypeConfig) -> dict[str, torch.dtype]:
    """Convert the parameters the configuration names; returns what was changed."""
    from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding
    from ..layers.layernorm import RMSNorm
    from ..layers.linear import LinearBase
    changed = {}
    for mod_name, mod in model.named_modules():
        if isinstance(mod, LinearBase):
            if getattr(mod, "qweight", None) is not None:
                continue                                  # quantised storage has its own dtype
        elif not isinstance(mod, (RMSNorm, VocabParallelEmbedding, ParallelLMHead)) \
                and type(mod).__name__ not in ("GemmaRMSNorm", "GatedRMSNorm"):
            continue
        for pname, p in mod.named_parameters(recurse=False):
            full = f"{mod_name}.{pname}" if mod_name else pname
            want = cfg.resolve(full)
            if want is not None and p.is_floating_point() and want.is_floating_point and p.dtype != want:
                p.data = p.data.to(want)
                changed[full] = want
    return changed
