"""Model configuration ingestion.

Reference: `python/sgl_jax/srt/configs/model_config.py:71-1034` (HF config, context length,
dtype, quantization, KV-head replication for `tp > kv_heads` :623-700, `MoEBackend` :36).
"""

from __future__ import annotations

import json
import os
from enum import Enum
from types import SimpleNamespace
from typing import Any

import torch

_DTYPES = {"half": torch.float16, "float16": torch.float16, "bfloat16": torch.bfloat16,
           "float": torch.float32, "float32": torch.float32}


class MoEBackend(Enum):
    EPMOE = "epmoe"
    FUSED = "fused"
    FUSED_V2 = "fused_v2"
    AUTO = "auto"


class AttentionArch(Enum):
    MHA = 1
    MLA = 2


class ConfigNS(SimpleNamespace):
    """HF-config-like attribute bag (used when `transformers` cannot parse a config)."""

    def to_dict(self):
        return dict(self.__dict__)

    def get(self, k, d=None):
        return getattr(self, k, d)


def load_hf_config(model_path: str, trust_remote_code: bool = False, revision: str | None = None,
                   override: dict | None = None):
    cfg_file = os.path.join(model_path, "config.json")
    if os.path.isfile(cfg_file):
        with open(cfg_file) as f:
            d = json.load(f)
    else:
        from transformers import AutoConfig
        d = AutoConfig.from_pretrained(model_path, trust_remote_code=trust_remote_code, revision=revision).to_dict()
    if override:
        d.update(override)
    cfg = ConfigNS(**d)
    tc = d.get("text_config")
    if isinstance(tc, dict):
        cfg.text_config = ConfigNS(**tc)
    return cfg


# target architecture -> class that loads its MTP / NextN layers as a draft model
_NEXTN_ARCH = {
    "MiMoForCausalLM": "MiMoMTP",
    "DeepseekV3ForCausalLM": "DeepseekV3ForCausalLMNextN",
    "MiMoV2FlashForCausalLM": "MiMoV2NextN",
    "MiMoV2ProForCausalLM": "MiMoV2NextN",
    "MiMoV2ForCausalLM": "MiMoV2NextN",
    "Glm4MoeForCausalLM": "Glm4MoeForCausalLMNextN",
}


class ModelConfig:
    def __init__(self, model_path: str, hf_config=None, dtype: str = "auto", context_length: int | None = None,
                 trust_remote_code: bool = False, revision: str | None = None, quantization: str | None = None,
                 model_override_args: str | dict | None = None, is_embedding: bool = False,
                 model_layer_nums: int | None = None, moe_backend: str = "epmoe", ep_size: int = 1,
                 is_draft_model: bool = False, download_dir: str | None = None, dtype_config=None):
        if isinstance(model_path, str) and not os.path.isdir(model_path) and hf_config is None:
            from ..utils.hf_transformers_utils import resolve_model_path
            model_path = resolve_model_path(model_path, download_dir, revision)
        self.model_path = model_path
        override = json.loads(model_override_args) if isinstance(model_override_args, str) else (model_override_args or {})
        self.hf_config = hf_config if hf_config is not None else load_hf_config(
            model_path, trust_remote_code, revision, override)
        if hf_config is not None and override:
            for k, v in override.items():
                setattr(self.hf_config, k, v)
        self.hf_text_config = getattr(self.hf_config, "text_config", None) or self.hf_config
        c = self.hf_text_config
        if model_layer_nums:
            c.num_hidden_layers = model_layer_nums
        self.is_embedding = is_embedding
        self.is_draft_model = is_draft_model
        self.architectures = list(getattr(self.hf_config, "architectures", None) or ["LlamaForCausalLM"])
        if is_draft_model:
            # multi-token-prediction heads live in the target checkpoint under their own class
            self.architectures = [_NEXTN_ARCH.get(a, a) for a in self.architectures]
        self.quantization = quantization
        self.moe_backend = MoEBackend(moe_backend)
        self.ep_size = ep_size

        self.hidden_size = c.hidden_size
        self.num_hidden_layers = c.num_hidden_layers
        self.num_attention_heads = c.num_attention_heads
        self.num_key_value_heads = getattr(c, "num_key_value_heads", None) or c.num_attention_heads
        self.head_dim = getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads
        self.vocab_size = c.vocab_size
        self.attention_arch = AttentionArch.MHA
        if getattr(c, "kv_lora_rank", None) and any("Deepseek" in a or "DeepSeek" in a or "Kimi" in a or "Glm5" in a or "GlmMoeDsa" in a
                                                    for a in self.architectures):
            self.attention_arch = AttentionArch.MLA
            self.kv_lora_rank = c.kv_lora_rank
            self.qk_rope_head_dim = c.qk_rope_head_dim
            self.qk_nope_head_dim = c.qk_nope_head_dim
            self.v_head_dim = c.v_head_dim
            self.head_dim = c.qk_nope_head_dim + c.qk_rope_head_dim
        derived = getattr(c, "max_position_embeddings", None) or getattr(c, "seq_length", 2048)
        rs = getattr(c, "rope_scaling", None)
        if isinstance(rs, dict) and rs.get("factor") and rs.get("rope_type", rs.get("type")) in ("yarn", "deepseek_yarn") \
                and rs.get("original_max_position_embeddings"):
            derived = max(derived, int(rs["original_max_position_embeddings"] * rs["factor"]))
        if context_length is not None:
            if context_length > derived and not os.environ.get("SGLANG_ALLOW_OVERWRITE_LONGER_CONTEXT_LEN"):
                raise ValueError(f"context_length {context_length} exceeds the model's {derived}; set "
                                 f"SGLANG_ALLOW_OVERWRITE_LONGER_CONTEXT_LEN=1 to force")
            self.context_len = context_length
        else:
            self.context_len = derived
        # positions up to context_len must exist in the rope table
        if getattr(c, "max_position_embeddings", 0) < self.context_len:
            c.max_position_embeddings = self.context_len

        if dtype == "auto":
            td = getattr(c, "torch_dtype", None) or getattr(c, "dtype", None) or "bfloat16"
            td = str(td).replace("torch.", "")
            self.dtype = _DTYPES.get(td, torch.bfloat16)
            if self.dtype == torch.float32 and not os.environ.get("SGLANG_KEEP_FP32"):
                self.dtype = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        else:
            self.dtype = _DTYPES[dtype]
        # per-module parameter dtypes (`--dtype-config`: a JSON object, a file, or a ready `DtypeConfig`)
        from .dtype_config import DtypeConfig
        self.dtype_config = dtype_config if isinstance(dtype_config, DtypeConfig) or dtype_config is None \
            else DtypeConfig.from_arg(dtype_config, self.dtype)

        eos = getattr(c, "eos_token_id", None)
        self.hf_eos_token_id = set(eos) if isinstance(eos, (list, tuple)) else ({eos} if eos is not None else set())
        self.sliding_window = getattr(c, "sliding_window", None) if getattr(c, "use_sliding_window", True) else None
        self.is_hybrid_swa = bool(getattr(c, "layer_types", None) and "sliding_attention" in c.layer_types
                                  and "full_attention" in c.layer_types)
        self.num_experts = getattr(c, "num_experts", None) or getattr(c, "n_routed_experts", None) or \
            getattr(c, "num_local_experts", None)

    @classmethod
    def from_server_args(cls, sa, model_path: str | None = None, **kw) -> "ModelConfig":
        # a draft model has its own revision (`--speculative-draft-model-revision`)
        revision = (getattr(sa, "speculative_draft_model_revision", None) or sa.revision) if kw.get("is_draft_model") \
            else sa.revision
        kw.setdefault("download_dir", getattr(sa, "download_dir", None))
        if not kw.get("is_draft_model"):
            kw.setdefault("dtype_config", getattr(sa, "dtype_config", None))
        return cls(model_path or sa.model_path, dtype=sa.dtype, context_length=sa.context_length,
                   trust_remote_code=sa.trust_remote_code, revision=revision, quantization=sa.quantization,
                   model_override_args=sa.json_model_override_args, is_embedding=sa.is_embedding,
                   model_layer_nums=sa.model_layer_nums, moe_backend=sa.moe_backend, ep_size=sa.ep_size, **kw)

    # KV heads owned by one tensor rank (replicated when tp > kv_heads)
    def get_num_kv_heads(self, tp: int) -> int:
        return max(1, self.num_key_value_heads // tp)

    def get_total_num_kv_heads_with_replication(self, tp: int) -> int:
        return max(self.num_key_value_heads, tp) if tp > self.num_key_value_heads else self.num_key_value_heads

    def needs_kv_head_replication(self, tp: int) -> bool:
        return tp > self.num_key_value_heads

    def get_num_attention_heads(self, tp: int) -> int:
        return self.num_attention_heads // tp
