"""Grammar backends for constrained decoding.

Reference: `python/sgl_jax/srt/constrained/base_grammar_backend.py` (async thread-pool compile,
cache keyed by (kind, spec), `INVALID_GRAMMAR_OBJ`) and `llguidance_backend.py`
(json / regex / ebnf / structural_tag)."""

from __future__ import annotations

import json
import logging
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass
from threading import Lock

import numpy as np

logger = logging.getLogger(__name__)


class BaseGrammarObject:
    is_invalid = False

    def __init__(self):
        self.finished = False

    def accept_token(self, token: int) -> None:
        raise NotImplementedError

    def fill_vocab_mask(self, mask: np.ndarray, idx: int) -> None:
        raise NotImplementedError

    def is_terminated(self) -> bool:
        return False

    def copy(self) -> "BaseGrammarObject":
        return self


class InvalidGrammarObject(BaseGrammarObject):
    is_invalid = True

    def __init__(self, error: str = ""):
        super().__init__()
        self.error = error


INVALID_GRAMMAR_OBJ = InvalidGrammarObject()


class BaseGrammarBackend:
    def __init__(self, num_threads: int = 4):
        self.executor = ThreadPoolExecutor(max_workers=num_threads)
        self.cache: dict[tuple[str, str], BaseGrammarObject] = {}
        self.lock = Lock()

    def dispatch(self, key: tuple[str, str]) -> BaseGrammarObject:
        kind, spec = key
        try:
            fn = {"json": self.dispatch_json, "regex": self.dispatch_regex, "ebnf": self.dispatch_ebnf,
                  "structural_tag": self.dispatch_structural_tag}[kind]
        except KeyError:
            return InvalidGrammarObject(f"unknown grammar kind {kind}")
        try:
            return fn(spec)
        except Exception as e:
            logger.warning("grammar compile failed for %s: %s", kind, e)
            return InvalidGrammarObject(str(e))

    def dispatch_json(self, spec): raise NotImplementedError
    def dispatch_regex(self, spec): raise NotImplementedError
    def dispatch_ebnf(self, spec): raise NotImplementedError
    def dispatch_structural_tag(self, spec): raise NotImplementedError

    def get_cached_or_future_value(self, key: tuple[str, str]):
        """Returns (object-or-future, cache_hit)."""
        with self.lock:
            v = self.cache.get(key)
        if v is not None:
            return (v.copy() if not v.is_invalid else v), True
        return self.executor.submit(self.dispatch, key), False

    def set_cache(self, key, value: BaseGrammarObject):
        with self.lock:
            self.cache[key] = value

    def reset(self):
        with self.lock:
            self.cache.clear()


class LLGuidanceGrammar(BaseGrammarObject):
    def __init__(self, matcher_factory, vocab_words: int):
        super().__init__()
        self._factory = matcher_factory
        self.matcher = matcher_factory()
        self.vocab_words = vocab_words

    def accept_token(self, token: int) -> None:
        if not self.matcher.is_stopped():
            self.matcher.consume_token(int(token))

    def fill_vocab_mask(self, mask: np.ndarray, idx: int) -> None:
        import llguidance.numpy as llnp
        if self.matcher.is_stopped():
            return
        llnp.fill_next_token_bitmask(self.matcher, mask, idx)

    def is_terminated(self) -> bool:
        return self.matcher.is_stopped()

    def copy(self):
        return LLGuidanceGrammar(self._factory, self.vocab_words)


class LLGuidanceBackend(BaseGrammarBackend):
    def __init__(self, tokenizer, vocab_size: int, whitespace_pattern: str | None = None,
                 any_whitespace: bool = True):
        super().__init__()
        import llguidance
        import llguidance.hf
        self.llg = llguidance
        self.vocab_size = vocab_size
        self.tokenizer = tokenizer
        self.llg_tokenizer = llguidance.hf.from_tokenizer(tokenizer, n_vocab=vocab_size)
        self.whitespace_pattern = whitespace_pattern
        self.any_whitespace = any_whitespace

    def _make(self, grammar: str) -> BaseGrammarObject:
        llg = self.llg
        err = llg.LLMatcher.validate_grammar(grammar, self.llg_tokenizer)
        if err:
            return InvalidGrammarObject(err)
        tok = self.llg_tokenizer
        return LLGuidanceGrammar(lambda: llg.LLMatcher(tok, grammar), (self.vocab_size + 31) // 32)

    def dispatch_json(self, spec: str):
        defaults = {}
        if self.whitespace_pattern:
            defaults["whitespace_pattern"] = self.whitespace_pattern
        elif not self.any_whitespace:
            defaults["whitespace_flexible"] = False
        return self._make(self.llg.LLMatcher.grammar_from_json_schema(spec, defaults=defaults or None))

    def dispatch_regex(self, spec: str):
        return self._make(self.llg.grammar_from("regex", spec))

    def dispatch_ebnf(self, spec: str):
        try:
            return self._make(self.llg.grammar_from("ebnf", spec))
        except Exception:
            return self._make(self.llg.grammar_from("lark", spec))

    def dispatch_structural_tag(self, spec: str):
        tag = json.loads(spec)
        structures = tag.get("structures", [])
        triggers = tag.get("triggers", [])
        tags = [self.llg.StructTag(trigger=next((t for t in triggers if s["begin"].startswith(t)), s["begin"]),
                                   begin=s["begin"], grammar=s.get("schema", {}), end=s["end"]) for s in structures]
        return self._make(self.llg.StructTag.to_grammar(tags))


class AllowListGrammar(BaseGrammarObject):
    """Minimal grammar used by tests and as a fallback: a fixed sequence of allowed-token sets."""

    def __init__(self, steps: list[set[int]], eos: int | None = None):
        super().__init__()
        self.steps = steps
        self.pos = 0
        self.eos = eos

    def accept_token(self, token: int) -> None:
        self.pos += 1

    def fill_vocab_mask(self, mask: np.ndarray, idx: int) -> None:
        from .bitmask_ops import fill_bitmask_from_allowed
        if self.pos < len(self.steps):
            fill_bitmask_from_allowed(mask, idx, self.steps[self.pos])
        elif self.eos is not None:
            fill_bitmask_from_allowed(mask, idx, {self.eos})

    def is_terminated(self) -> bool:
        return self.pos >= len(self.steps)

    def copy(self):
        return AllowListGrammar(self.steps, self.eos)


def create_grammar_backend(server_args, tokenizer, vocab_size: int):
    name = server_args.grammar_backend
    if name in (None, "none"):
        return None
    if name == "llguidance":
        try:
            return LLGuidanceBackend(tokenizer, vocab_size, server_args.constrained_json_whitespace_pattern,
                                     not server_args.constrained_json_disable_any_whitespace)
        except Exception as e:
            logger.warning("llguidance backend unavailable (%s): constrained decoding disabled", e)
            return None
    raise ValueError(f"Invalid grammar backend: {name}")
