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


def resolve_model_path(model_path: str, download_dir: str | None = None, revision: str | None = None) -> str:
    """A local directory is used as is; anything else is taken as a hub repository id and fetched once into
    `download_dir` (`--download-dir`, default: the hub cache) at `revision` (reference `model_loader/loader.py`,
    `configs/load_config.py` `download_dir`).  Only the files a server needs are fetched."""
    import os
    if model_path is None or os.path.isdir(model_path):
        return model_path
    try:
        from huggingface_hub import snapshot_download
    except ImportError as e:
        raise FileNotFoundError(f"{model_path} is not a local directory and huggingface_hub is not installed") from e
    return snapshot_download(model_path, cache_dir=download_dir, revision=revision,
                             allow_patterns=["*.json", "*.safetensors", "*.model", "*.txt", "*.tiktoken", "*.jinja"])

