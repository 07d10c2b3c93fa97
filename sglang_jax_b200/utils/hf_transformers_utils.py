"""Tokenizer / config / processor loading (reference `python/sgl_jax/srt/hf_transformers_utils.py`:
`get_config` :112, `get_tokenizer` :255, `get_processor` :482)."""

from __future__ import annotations

import os


def get_tokenizer(tokenizer_path: str, tokenizer_mode: str = "auto", trust_remote_code: bool = False,
                  revision: str | None = None, tokenizer_backend: str = "huggingface", **kw):
    if tokenizer_backend == "tiktoken" or tokenizer_path.endswith(".tiktoken") or tokenizer_path.endswith(".json") \
            and os.path.basename(tokenizer_path).startswith("tiktoken"):
        from .tiktoken_tokenizer import TiktokenTokenizer
        return TiktokenTokenizer(tokenizer_path)
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(tokenizer_path, trust_remote_code=trust_remote_code, revision=revision,
                                        use_fast=(tokenizer_mode != "slow"), **kw)
    attach_additional_stop_token_ids(tok)
    return tok


def attach_additional_stop_token_ids(tokenizer):
    added = getattr(tokenizer, "get_added_vocab", lambda: {})()
    if "<|eom_id|>" in added:
        tokenizer.additional_stop_token_ids = {added["<|eom_id|>"]}
    else:
        tokenizer.additional_stop_token_ids = None


def get_config(model_path: str, trust_remote_code: bool = False, revision: str | None = None,
               model_override_args: dict | None = None):
    from ..configs.model_config import load_hf_config
    return load_hf_config(model_path, trust_remote_code, revision, model_override_args)


def get_processor(model_path: str, trust_remote_code: bool = False, revision: str | None = None, **kw):
    from transformers import AutoProcessor
    return AutoProcessor.from_pretrained(model_path, trust_remote_code=trust_remote_code, revision=revision, **kw)


def get_context_length(config) -> int:
    for k in ("max_sequence_length", "seq_length", "max_seq_len", "model_max_length", "max_position_embeddings"):
        v = getattr(config, k, None)
        if v is not None:
            return int(v)
    return 2048
