"""Shared pieces of the accuracy evaluations (reference `test/srt/eval/simple_eval_common.py`): a
sampler that talks to a running server's OpenAI chat endpoint (or to an in-process `Engine`), a
thread-pool map, result aggregation and the answer-extraction patterns."""

from __future__ import annotations

import dataclasses
import re
import statistics
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Callable

ANSWER_PATTERN_MULTICHOICE = r"(?i)Answer\s*:\s*\$?([A-D])\$?"
ANSWER_PATTERN = r"(?i)Answer\s*:\s*([^\n]+)"
QUERY_TEMPLATE_MULTICHOICE = """
Answer the following multiple choice question. The last line of your response should be of the following format: 'Answer: $LETTER' (without quotes) where LETTER is one of ABCD. Think step by step before answering.

{Question}

A) {A}
B) {B}
C) {C}
D) {D}
""".strip()


@dataclasses.dataclass
class SingleEvalResult:
    score: float | None
    metrics: dict[str, float] = dataclasses.field(default_factory=dict)
    convo: list | None = None


@dataclasses.dataclass
class EvalResult:
    score: float | None
    metrics: dict[str, float]
    convos: list


class SamplerBase:
    def __call__(self, messages: list[dict]) -> str:
        raise NotImplementedError


class ChatCompletionSampler(SamplerBase):
    """`POST {base_url}/v1/chat/completions`; retries transient failures with back-off."""

    def __init__(self, base_url: str, model: str = "default", temperature: float = 0.0, max_tokens: int = 2048,
                 system_message: str | None = None, api_key: str | None = None, timeout: float = 600, retries: int = 4):
        self.url = base_url.rstrip("/") + "/v1/chat/completions"
        self.model, self.temperature, self.max_tokens = model, temperature, max_tokens
        self.system_message, self.api_key, self.timeout, self.retries = system_message, api_key, timeout, retries

    def __call__(self, messages):
        import time

        import requests
        if self.system_message:
            messages = [{"role": "system", "content": self.system_message}] + list(messages)
        body = {"model": self.model, "messages": messages, "temperature": self.temperature, "max_tokens": self.max_tokens}
        headers = {"Authorization": f"Bearer {self.api_key}"} if self.api_key else {}
        for attempt in range(self.retries + 1):
            try:
                r = requests.post(self.url, json=body, headers=headers, timeout=self.timeout)
                r.raise_for_status()
                return r.json()["choices"][0]["message"]["content"] or ""
            except Exception:
                if attempt == self.retries:
                    return ""
                time.sleep(2 ** attempt)


class EngineSampler(SamplerBase):
    """In-process `Engine` with a chat template applied by its tokenizer."""

    def __init__(self, engine, temperature: float = 0.0, max_tokens: int = 2048):
        self.engine, self.temperature, self.max_tokens = engine, temperature, max_tokens

    def __call__(self, messages):
        tok = self.engine.tokenizer_manager.tokenizer
        if hasattr(tok, "apply_chat_template"):
            prompt = tok.apply_chat_template(messages, tokenize=False, add_generation_prompt=True)
        else:
            prompt = "\n".join(f"{m['role']}: {m['content']}" for m in messages) + "\nassistant:"
        out = self.engine.generate(prompt, {"temperature": self.temperature, "max_new_tokens": self.max_tokens})
        return out["text"]


class Eval:
    def __call__(self, sampler: SamplerBase) -> EvalResult:
        raise NotImplementedError


def map_with_progress(fn: Callable, xs: list, num_threads: int = 32) -> list:
    if num_threads <= 1:
        return [fn(x) for x in xs]
    with ThreadPoolExecutor(num_threads) as ex:
        return list(ex.map(fn, xs))


def aggregate_results(results: list[SingleEvalResult]) -> EvalResult:
    by_name: dict[str, list[float]] = {}
    for r in results:
        for k, v in r.metrics.items():
            by_name.setdefault(k, []).append(v)
        if r.score is not None:
            by_name.setdefault("score", []).append(r.score)
    metrics = {}
    for k, vs in by_name.items():
        metrics[k] = statistics.fmean(vs)
        if len(vs) > 1:
            metrics[k + ":std"] = statistics.pstdev(vs)
    return EvalResult(metrics.pop("score", None), metrics, [r.convo for r in results])


def normalize_number(s: str) -> str:
    s = s.strip().replace(",", "").replace("$", "").rstrip(".")
    m = re.findall(r"-?\d+(?:\.\d+)?", s)
    if not m:
        return s.strip().lower()
    x = m[-1]
    return x[:-2] if x.endswith(".0") else x


def make_report(result: EvalResult) -> str:
    lines = [f"score: {result.score:.4f}" if result.score is not None else "score: n/a"]
    lines += [f"{k}: {v:.4f}" for k, v in sorted(result.metrics.items())]
    return "\n".join(lines)
