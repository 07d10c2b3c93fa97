"""GSM8K / MGSM-style numeric answers (reference `test/srt/eval/simple_eval_gsm8k.py`, `benchmark/gsm8k`):
JSONL rows `{"question": ..., "answer": "... #### 42"}`; few-shot examples are the first rows."""

from __future__ import annotations

import json
import re

from .simple_eval_common import ANSWER_PATTERN, Eval, SingleEvalResult, aggregate_results, map_with_progress, normalize_number

INSTRUCTION = ("Solve this math problem. Give the reasoning steps before giving the final answer on the last line by "
               "itself in the format of \"Answer:\". Do not add anything other than the number after \"Answer:\".")


def gold(answer: str) -> str:
    return normalize_number(answer.split("####")[-1])


class GSM8KEval(Eval):
    def __init__(self, data_path: str, num_examples: int | None = None, num_shots: int = 5, num_threads: int = 32):
        with open(data_path) as f:
            rows = [json.loads(l) for l in f if l.strip()]
        self.shots, rest = rows[:num_shots], rows[num_shots:]
        self.examples = rest[:num_examples] if num_examples else rest
        self.num_threads = num_threads

    def _few_shot(self) -> str:
        return "".join(f"Question: {r['question']}\nAnswer: {gold(r['answer'])}\n\n" for r in self.shots)

    def __call__(self, sampler):
        head = self._few_shot()

        def one(row):
            prompt = [{"role": "user", "content": f"{INSTRUCTION}\n\n{head}Question: {row['question']}"}]
            text = sampler(prompt) or ""
            m = re.findall(ANSWER_PATTERN, text)
            pred = normalize_number(m[-1]) if m else normalize_number(text[-64:])
            score = 1.0 if pred == gold(row["answer"]) else 0.0
            return SingleEvalResult(score, {"invalid": 0.0 if m else 1.0}, prompt + [{"role": "assistant", "content": text}])
        return aggregate_results(map_with_progress(one, self.examples, self.num_threads))
