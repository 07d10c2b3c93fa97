"""Per-request sampling parameters.

Same constructor keywords, normalisation and validation rules as the reference's
`SamplingParams` (`python/sgl_jax/srt/sampling/sampling_params.py:9-167`):
a temperature below 1e-6 is rewritten to greedy (`top_k = 1`), `top_k = -1`
means the whole vocabulary.
"""

from __future__ import annotations

import os

_SAMPLING_EPS = 1e-6
TOP_K_ALL = 1 << 30
DEFAULT_SAMPLING_SEED = 42

_FIELDS = (
    "max_new_tokens", "stop", "stop_token_ids", "temperature", "top_p", "top_k", "min_p",
    "frequency_penalty", "presence_penalty", "repetition_penalty", "min_new_tokens", "n",
    "json_schema", "regex", "ebnf", "structural_tag", "ignore_eos", "skip_special_tokens",
    "spaces_between_special_tokens", "no_stop_trim", "stream_interval", "logit_bias",
    "sampling_seed",
)


class SamplingParams:
    def __init__(
        self,
        max_new_tokens: int = 128,
        stop: str | list[str] | None = None,
        stop_token_ids: list[int] | None = None,
        temperature: float = 1.0,
        top_p: float = 1.0,
        top_k: int = -1,
        min_p: float = 0.0,
        frequency_penalty: float = 0.0,
        presence_penalty: float = 0.0,
        repetition_penalty: float = 1.0,
        min_new_tokens: int = 0,
        n: int = 1,
        json_schema: str | None = None,
        regex: str | None = None,
        ebnf: str | None = None,
        structural_tag: str | None = None,
        ignore_eos: bool = False,
        skip_special_tokens: bool = True,
        spaces_between_special_tokens: bool = True,
        no_stop_trim: bool = False,
        stream_interval: int | None = None,
        logit_bias: dict[str, float] | None = None,
        sampling_seed: int | None = None,
    ) -> None:
        self.max_new_tokens = max_new_tokens
        self.stop_strs = stop
        self.stop_token_ids = set(stop_token_ids) if stop_token_ids else None
        self.temperature = temperature
        self.top_p = top_p
        self.top_k = top_k
        self.min_p = min_p
        self.frequency_penalty = frequency_penalty
        self.presence_penalty = presence_penalty
        self.repetition_penalty = repetition_penalty
        self.min_new_tokens = min_new_tokens
        self.n = n
        self.json_schema = json_schema
        self.regex = regex
        self.ebnf = ebnf
        self.structural_tag = structural_tag
        self.ignore_eos = ignore_eos
        self.skip_special_tokens = skip_special_tokens
        self.spaces_between_special_tokens = spaces_between_special_tokens
        self.no_stop_trim = no_stop_trim
        self.stream_interval = stream_interval
        self.logit_bias = logit_bias
        if sampling_seed is None and os.environ.get(
                "SGLANG_ENABLE_DETERMINISTIC_SAMPLING", "").lower() in ("1", "true"):
            sampling_seed = DEFAULT_SAMPLING_SEED
        self.sampling_seed = sampling_seed
        self.stop_str_max_len = 0

        if 0 <= self.temperature < _SAMPLING_EPS:
            self.temperature = 1.0
            self.top_k = 1
        if self.top_k == -1:
            self.top_k = TOP_K_ALL

    @property
    def is_greedy(self) -> bool:
        return self.top_k == 1

    @property
    def has_grammar(self) -> bool:
        return any(x is not None for x in (self.json_schema, self.regex, self.ebnf, self.structural_tag))

    def verify(self, vocab_size: int) -> None:
        def bad(msg):
            raise ValueError(msg)

        if self.temperature < 0.0:
            bad(f"temperature must be non-negative, got {self.temperature}.")
        if not 0.0 < self.top_p <= 1.0:
            bad(f"top_p must be in (0, 1], got {self.top_p}.")
        if not 0.0 <= self.min_p <= 1.0:
            bad(f"min_p must be in [0, 1], got {self.min_p}.")
        if self.top_k < 1:
            bad(f"top_k must be -1 (disable) or at least 1, got {self.top_k}.")
        for name in ("frequency_penalty", "presence_penalty"):
            v = getattr(self, name)
            if not -2.0 <= v <= 2.0:
                bad(f"{name} must be in [-2, 2], got {v}.")
        if not 0.0 <= self.repetition_penalty <= 2.0:
            bad(f"repetition_penalty must be in [0, 2], got {self.repetition_penalty}.")
        if self.min_new_tokens < 0:
            bad(f"min_new_tokens must be in [0, max_new_tokens], got {self.min_new_tokens}.")
        if self.max_new_tokens is not None:
            if self.max_new_tokens < 0:
                bad(f"max_new_tokens must be at least 0, got {self.max_new_tokens}.")
            if self.min_new_tokens > self.max_new_tokens:
                bad(f"min_new_tokens must be in [0, max_new_tokens({self.max_new_tokens})], "
                    f"got {self.min_new_tokens}.")
        if self.logit_bias is not None:
            for token_id in self.logit_bias:
                if not 0 <= int(token_id) < vocab_size:
                    bad(f"logit_bias must has keys in [0, {vocab_size - 1}], got {token_id}.")
        if sum(x is not None for x in (self.json_schema, self.regex, self.ebnf)) > 1:
            bad("Only one of regex, json_schema, or ebnf can be set.")

    def normalize(self, tokenizer) -> None:
        if self.stop_strs is None:
            self.stop_strs = []
            self.stop_str_max_len = 0
            return
        if isinstance(self.stop_strs, str):
            self.stop_strs = [self.stop_strs]
        m = 0
        for s in self.stop_strs:
            m = max(m, len(tokenizer.encode(s, add_special_tokens=False)) if tokenizer is not None else len(s))
        self.stop_str_max_len = m

    def convert_to_dict(self) -> dict:
        out = {}
        for k, v in self.__dict__.items():
            if k.startswith("_") or k == "stop_str_max_len":
                continue
            if k == "stop_token_ids":
                out[k] = list(v) if v is not None else None
            elif k == "stop_strs":
                out["stop"] = v
            else:
                out[k] = v
        if out.get("top_k") == TOP_K_ALL:
            out["top_k"] = -1
        return out

    @classmethod
    def from_dict(cls, d: dict | None) -> "SamplingParams":
        d = dict(d or {})
        if "stop_strs" in d:
            d["stop"] = d.pop("stop_strs")
        return cls(**{k: v for k, v in d.items() if k in _FIELDS})

    def __repr__(self):
        return f"SamplingParams({self.convert_to_dict()})"
