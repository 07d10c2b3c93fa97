"""MMLU (reference `test/srt/eval/simple_eval_mmlu.py`): rows `Question,A,B,C,D,Answer,Subject` from a
local CSV; zero-shot chain-of-thought prompt; the letter after "Answer:" is scored."""

from __future__ import annotations

import csv
import random
import re

from .simple_eval_common import (ANSWER_PATTERN_MULTICHOICE, QUERY_TEMPLATE_MULTICHOICE, Eval, SingleEvalResult,
                                 aggregate_results, map_with_progress)

SUBJECT_TO_CATEGORY = {"abstract_algebra": "stem", "college_physics": "stem", "computer_security": "stem",
                       "machine_learning": "stem", "philosophy": "humanities", "world_religions": "humanities",
                       "econometrics": "social_sciences", "sociology": "social_sciences", "anatomy": "other",
                       "marketing": "other"}


class MMLUEval(Eval):
    def __init__(self, data_path: str, num_examples: int | None = None, num_threads: int = 32, seed: int = 0):
        with open(data_path, newline="") as f:
            rows = list(csv.DictReader(f))
        if num_examples:
            rows = random.Random(seed).sample(rows, min(num_examples, len(rows)))
        self.examples, self.num_threads = rows, num_threads

    def __call__(self, sampler):
        def one(row):
            prompt = [{"role": "user", "content": QUERY_TEMPLATE_MULTICHOICE.format(**row)}]
            text = sampler(prompt)
            m = re.search(ANSWER_PATTERN_MULTICHOICE, text or "")
            score = 1.0 if m and m.group(1).upper() == row["Answer"].strip().upper() else 0.0
            cat = SUBJECT_TO_CATEGORY.get(row.get("Subject", ""), "other")
            return SingleEvalResult(score, {cat: score}, prompt + [{"role": "assistant", "content": text}])
        return aggregate_results(map_with_progress(one, self.examples, self.num_threads))
