"""Adapter that makes a `tiktoken` BPE file usable where a HF tokenizer is expected (reference
`hf_transformers_utils.get_tokenizer` tiktoken branch, `python/sgl_jax/srt/hf_transformers_utils.py:255`)."""

from __future__ import annotations

import base64
import json
import os

PAT = r"""'(?i:[sdmt]|ll|ve|re)|[^\r\n\p{L}\p{N}]?+\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]++[\r\n]*|\s*[\r\n]|\s+(?!\S)|\s+"""


class TiktokenTokenizer:
    def __init__(self, path: str, special_tokens: list[str] | None = None, eos_token: str = "<|endoftext|>",
                 chat_template: str | None = None):
        import tiktoken
        ranks = {}
        with open(path, "rb") as f:
            for line in f:
                if line.strip():
                    tok, rank = line.split()
                    ranks[base64.b64decode(tok)] = int(rank)
        specials = list(special_tokens or [eos_token])
        cfg = os.path.join(os.path.dirname(path), "tokenizer_config.json")
        if os.path.exists(cfg):
            with open(cfg) as f:
                c = json.load(f)
            chat_template = chat_template or c.get("chat_template")
            for t in c.get("additional_special_tokens", []):
                if t not in specials:
                    specials.append(t)
        n = len(ranks)
        self.special = {t: n + i for i, t in enumerate(specials)}
        self.enc = tiktoken.Encoding(name=os.path.basename(path), pat_str=PAT, mergeable_ranks=ranks,
                                     special_tokens=self.special)
        self.eos_token = eos_token
        self.eos_token_id = self.special.get(eos_token)
        self.pad_token_id = self.eos_token_id
        self.bos_token_id = None
        self.vocab_size = n + len(specials)
        self.chat_template = chat_template
        self.additional_stop_token_ids = set()

    def __len__(self):
        return self.vocab_size

    def encode(self, text: str, add_special_tokens: bool = False, **kw) -> list[int]:
        return self.enc.encode(text, allowed_special="all")

    def __call__(self, text, **kw):
        if isinstance(text, str):
            return {"input_ids": self.encode(text)}
        return {"input_ids": [self.encode(t) for t in text]}

    def decode(self, ids, skip_special_tokens: bool = True, **kw) -> str:
        ids = [int(i) for i in ids]
        if skip_special_tokens:
            sp = set(self.special.values())
            ids = [i for i in ids if i not in sp]
        return self.enc.decode(ids)

    def batch_decode(self, batch, **kw) -> list[str]:
        return [self.decode(x, **kw) for x in batch]

    def convert_ids_to_tokens(self, ids):
        return [self.enc.decode_single_token_bytes(int(i)).decode("utf-8", errors="replace") for i in ids]

    def apply_chat_template(self, messages, tokenize: bool = True, add_generation_prompt: bool = True,
                            chat_template: str | None = None, **kw):
        from ..conversation import generate_chat_conv
        from ..jinja_template_utils import render_template
        tpl = chat_template or self.chat_template
        text = render_template(tpl, messages=messages, add_generation_prompt=add_generation_prompt, **kw) if tpl \
            else generate_chat_conv(messages, None, None, add_generation_prompt)
        return self.encode(text) if tokenize else text
