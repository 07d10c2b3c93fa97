"""Further accuracy evaluations (reference `test/srt/eval/`: `simple_eval_math.py`, `simple_eval_aime25.py` /
`simple_eval_aime26.py`, `simple_eval_gpqa.py`, `simple_eval_humaneval.py`, `simple_eval_mgsm.py`,
`simple_eval_csimpleqa.py`).  Every dataset is a local file (nothing is downloaded):

* MATH       CSV with columns `Question`, `Answer`; the model ends with a line `Answer: ...`; equality by normalised
             strings, or by asking a checker sampler when one is given
* AIME       JSONL rows `{"problem" | "question": ..., "answer": ...}`; answer inside `\\boxed{}`; integer compare
* GPQA       CSV with `Question`, `Correct Answer`, `Incorrect Answer 1..3`; options shuffled with a fixed seed
* HumanEval  JSONL rows `{"task_id", "prompt", "test", "entry_point"}`; the completion runs in a subprocess with a
             time limit; pass@1
* MGSM       TSV files `mgsm_<lang>.tsv` (`question <tab> answer`); language-specific instruction and answer prefix
* C-SimpleQA JSONL rows `{"question", "answer"}`; a grader sampler labels each reply A (correct), B (incorrect) or
             C (not attempted)
"""

from __future__ import annotations

import csv
import json
import os
import random
import re
import subprocess
import sys
import tempfile

from .simple_eval_common import (ANSWER_PATTERN, ANSWER_PATTERN_MULTICHOICE, QUERY_TEMPLATE_MULTICHOICE, Eval,
                                 SingleEvalResult, aggregate_results, map_with_progress, normalize_number)


def _user(text: str) -> list[dict]:
    return [{"role": "user", "content": text}]


# ------------------------------------------------------------------------------------------ MATH
MATH_TEMPLATE = ("Solve the following math problem step by step. The last line of your response should be of the form "
                 "Answer: $ANSWER (without quotes) where $ANSWER is the answer to the problem.\n\n{Question}\n\n"
                 "Remember to put your answer on its own line after \"Answer:\", and you do not need to use a \\boxed command.")

EQUALITY_TEMPLATE = ("Look at the following two expressions (answers to a math problem) and judge whether they are "
                     "equivalent. Only perform trivial simplifications.\n\n    Expression 1: {a}\n    Expression 2: {b}\n\n"
                     "Respond with only \"Yes\" or \"No\" (without quotes).")


def normalize_math(s: str | None) -> str:
    if s is None:
        return ""
    s = s.strip().strip("$").strip()
    s = re.sub(r"\\boxed\{(.*)\}$", r"\1", s)
    s = s.replace("\\left", "").replace("\\right", "").replace("\\!", "").replace("\\,", "").replace(" ", "")
    s = s.replace("dfrac", "frac").replace("tfrac", "frac").rstrip(".")
    s = re.sub(r"\\text\{([^}]*)\}", r"\1", s)
    if re.fullmatch(r"-?\d[\d,]*(\.\d+)?", s):
        s = normalize_number(s)
    return s.lower()


def check_equality(checker, a: str, b: str | None) -> bool:
    if b is None:
        return False
    if normalize_math(a) == normalize_math(b):
        return True
    if checker is None:
        return False
    return (checker(_user(EQUALITY_TEMPLATE.format(a=a, b=b))) or "").strip().lower().startswith("yes")


class MathEval(Eval):
    def __init__(self, data_path: str, num_examples: int | None = None, num_threads: int = 32, equality_checker=None):
        with open(data_path, newline="") as f:
            rows = list(csv.DictReader(f))
        self.examples = random.Random(0).sample(rows, num_examples) if num_examples and num_examples < len(rows) else rows
        self.num_threads, self.checker = num_threads, equality_checker

    def __call__(self, sampler):
        def one(row):
            prompt = _user(MATH_TEMPLATE.format(Question=row["Question"]))
            text = sampler(prompt) or ""
            m = re.findall(ANSWER_PATTERN, text)
            pred = m[-1] if m else None
            score = float(check_equality(self.checker, row["Answer"], pred))
            return SingleEvalResult(score, {"invalid": 0.0 if m else 1.0}, prompt + [{"role": "assistant", "content": text}])
        return aggregate_results(map_with_progress(one, self.examples, self.num_threads))


# ------------------------------------------------------------------------------------------ AIME
AIME_TEMPLATE = ("Solve the following math problem step by step. Put your answer inside \\boxed{{}}.\n\n{question}\n\n"
                 "Remember to put your answer inside \\boxed{{}}.")


def boxed_answer(text: str) -> str:
    """Content of the last `\\boxed{...}` (balanced braces)."""
    i = text.rfind("\\boxed{")
    if i < 0:
        return ""
    depth, out = 0, []
    for ch in text[i + len("\\boxed{") - 1:]:
        if ch == "{":
            depth += 1
            if depth == 1:
                continue
        elif ch == "}":
            depth -= 1
            if depth == 0:
                break
        out.append(ch)
    return "".join(out).strip()


def same_integer(target: str, pred: str) -> bool:
    t, p = normalize_number(str(target)), normalize_number(pred)
    try:
        return int(float(t)) == int(float(p))
    except ValueError:
        return t == p and t != ""


class AIMEEval(Eval):
    def __init__(self, data_path: str, num_examples: int | None = None, num_threads: int = 32):
        with open(data_path) as f:
            rows = [json.loads(l) for l in f if l.strip()]
        self.examples = rows[:num_examples] if num_examples else rows
        self.num_threads = num_threads

    def __call__(self, sampler):
        def one(row):
            q = row.get("problem") or row.get("question")
            prompt = _user(AIME_TEMPLATE.format(question=q))
            text = sampler(prompt) or ""
            pred = boxed_answer(text)
            return SingleEvalResult(float(same_integer(str(row["answer"]), pred)), {"invalid": 0.0 if pred else 1.0},
                                    prompt + [{"role": "assistant", "content": text}])
        return aggregate_results(map_with_progress(one, self.examples, self.num_threads))


# ------------------------------------------------------------------------------------------ GPQA
class GPQAEval(Eval):
    def __init__(self, data_path: str, num_examples: int | None = None, num_threads: int = 32, n_repeats: int = 1):
        with open(data_path, newline="") as f:
            rows = list(csv.DictReader(f))
        rng = random.Random(0)
        if num_examples and num_examples < len(rows):
            rows = rng.sample(rows, num_examples)
        rows = rows * n_repeats
        self.examples = [dict(r, permutation=rng.sample(range(4), 4)) for r in rows]
        self.num_threads = num_threads

    def __call__(self, sampler):
        def one(row):
            options = [row["Correct Answer"], row["Incorrect Answer 1"], row["Incorrect Answer 2"], row["Incorrect Answer 3"]]
            shuffled = [options[i] for i in row["permutation"]]
            correct = "ABCD"[shuffled.index(row["Correct Answer"])]
            prompt = _user(QUERY_TEMPLATE_MULTICHOICE.format(Question=row["Question"], A=shuffled[0], B=shuffled[1],
                                                             C=shuffled[2], D=shuffled[3]))
            text = sampler(prompt) or ""
            m = re.findall(ANSWER_PATTERN_MULTICHOICE, text)
            pred = m[-1].upper() if m else None
            return SingleEvalResult(1.0 if pred == correct else 0.0, {"invalid": 0.0 if m else 1.0},
                                    prompt + [{"role": "assistant", "content": text}])
        return aggregate_results(map_with_progress(one, self.examples, self.num_threads))


# ------------------------------------------------------------------------------------------ HumanEval
HUMANEVAL_INSTRUCTION = "Read the following function signature and docstring, and fully implement the function described. " \
                        "Your response should only contain the code for this function.\n"


def extract_code(completion: str) -> str:
    m = re.findall(r"```(?:python)?\n(.*?)```", completion, re.DOTALL)
    return m[0] if m else completion


def run_program(program: str, timeout: float = 10.0) -> bool:
    """True when the program exits 0 within the limit (own interpreter process, scratch working directory)."""
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "prog.py")
        with open(path, "w") as f:
            f.write(program)
        try:
            r = subprocess.run([sys.executable, "-I", path], cwd=d, capture_output=True, timeout=timeout)
            return r.returncode == 0
        except subprocess.TimeoutExpired:
            return False


class HumanEvalEval(Eval):
    def __init__(self, data_path: str, num_examples: int | None = None, num_threads: int = 16, timeout: float = 10.0):
        with open(data_path) as f:
            rows = [json.loads(l) for l in f if l.strip()]
        self.examples = rows[:num_examples] if num_examples else rows
        self.num_threads, self.timeout = num_threads, timeout

    def __call__(self, sampler):
        def one(row):
            prompt = _user(HUMANEVAL_INSTRUCTION + row["prompt"])
            text = sampler(prompt) or ""
            code = extract_code(text)
            # a full definition replaces the prompt's stub, a bare body is appended to it
            body = code if re.search(rf"def\s+{re.escape(row['entry_point'])}\s*\(", code) else row["prompt"] + code
            program = f"{body}\n\n{row['test']}\n\ncheck({row['entry_point']})\n"
            ok = run_program(program, self.timeout)
            return SingleEvalResult(1.0 if ok else 0.0, {"pass@1": 1.0 if ok else 0.0},
                                    prompt + [{"role": "assistant", "content": text}])
        return aggregate_results(map_with_progress(one, self.examples, self.num_threads))


# ------------------------------------------------------------------------------------------ MGSM
MGSM_LANG = {
    "en": ("Solve this math problem. Give the reasoning steps before giving the final answer on the last line by itself "
           "in the format of \"Answer:\". Do not add anything other than the integer answer after \"Answer:\".", "Answer"),
    "de": ("Löse dieses Mathematikproblem. Gib die Schritte zur Begründung an, bevor du die endgültige Antwort in der "
           "letzten Zeile alleine im Format \"Antwort:\" gibst. Füge nichts anderes als die ganzzahlige Antwort nach "
           "\"Antwort:\" hinzu.", "Antwort"),
    "fr": ("Résolvez ce problème de mathématiques. Donnez les étapes de raisonnement avant de fournir la réponse finale sur "
           "la dernière ligne elle-même dans le format de \"Réponse:\". N'ajoutez rien d'autre que la réponse entière après "
           "\"Réponse:\".", "Réponse"),
    "es": ("Resuelve este problema matemático. Proporciona los pasos de razonamiento antes de dar la respuesta final en la "
           "última línea por sí misma en el formato de \"Respuesta:\". No añadas nada más que la respuesta entera después de "
           "\"Respuesta:\".", "Respuesta"),
    "zh": ("解决这个数学问题。在最后一行给出答案前，请提供推理步骤。最后一行应该以 \"答案:\" 的形式独立给出答案。在 \"答案:\" 后不要添加除整数答案之外的任何内容。", "答案"),
    "ja": ("この数学の問題を解いてください。最終的な答えを出す前に、解答の推論過程を記述してください。そして最後の行には "
           "\"答え:\" の形式で答えを記述し、その後には整数の答え以外何も追加しないでください。", "答え"),
    "ru": ("Решите эту математическую задачу. Объясните шаги рассуждения перед тем, как дать окончательный ответ в последней "
           "строке сам по себе в формате \"Ответ:\". Не добавляйте ничего, кроме целочисленного ответа после \"Ответ:\".", "Ответ"),
}


def mgsm_answer(text: str, prefix: str) -> str:
    if prefix not in text:
        return ""
    tail = text.split(prefix)[-1].strip().lstrip(":：").strip()
    nums = re.findall(r"-?\d+(?:[.,]\d+)*", tail.replace(",", ""))
    return nums[-1].rstrip(".") if nums else ""


class MGSMEval(Eval):
    def __init__(self, data_dir: str, languages: list[str] | None = None, num_examples_per_lang: int | None = None,
                 num_threads: int = 32):
        self.examples = []
        for lang in languages or sorted(MGSM_LANG):
            path = os.path.join(data_dir, f"mgsm_{lang}.tsv")
            if not os.path.exists(path):
                continue
            with open(path, encoding="utf-8") as f:
                rows = [l.rstrip("\n").split("\t") for l in f if "\t" in l]
            for q, a in rows[:num_examples_per_lang] if num_examples_per_lang else rows:
                self.examples.append({"lang": lang, "question": q, "answer": a})
        self.num_threads = num_threads

    def __call__(self, sampler):
        def one(row):
            instruction, prefix = MGSM_LANG[row["lang"]]
            prompt = _user(f"{instruction}\n\n{row['question']}")
            text = sampler(prompt) or ""
            pred = mgsm_answer(text, prefix)
            ok = same_integer(row["answer"], pred) if pred else False
            return SingleEvalResult(float(ok), {row["lang"]: float(ok)}, prompt + [{"role": "assistant", "content": text}])
        return aggregate_results(map_with_progress(one, self.examples, self.num_threads))


# ------------------------------------------------------------------------------------------ C-SimpleQA
GRADER_TEMPLATE = """Grade the predicted answer to a factual question against the gold target as one of:
A: CORRECT (the prediction contains the gold target's information and nothing that contradicts it)
B: INCORRECT (the prediction contradicts the gold target)
C: NOT_ATTEMPTED (the prediction neither gives the gold target's information nor contradicts it)

Question: {question}
Gold target: {target}
Predicted answer: {predicted}

Reply with the single letter A, B or C."""


def parse_grade(text: str) -> str:
    m = re.search(r"\b([ABC])\b", text or "")
    return m.group(1) if m else "C"


class CSimpleQAEval(Eval):
    def __init__(self, data_path: str, grader, num_examples: int | None = None, num_threads: int = 32):
        with open(data_path, encoding="utf-8") as f:
            rows = [json.loads(l) for l in f if l.strip()]
        self.examples = rows[:num_examples] if num_examples else rows
        self.grader, self.num_threads = grader, num_threads

    def __call__(self, sampler):
        def one(row):
            prompt = _user(row["question"])
            text = sampler(prompt) or ""
            grade = parse_grade(self.grader(_user(GRADER_TEMPLATE.format(question=row["question"], target=row["answer"],
                                                                        predicted=text))))
            return SingleEvalResult(1.0 if grade == "A" else 0.0,
                                    {"is_correct": float(grade == "A"), "is_incorrect": float(grade == "B"),
                                     "is_not_attempted": float(grade == "C")},
                                    prompt + [{"role": "assistant", "content": text}])
        res = aggregate_results(map_with_progress(one, self.examples, self.num_threads))
        c, i = res.metrics.get("is_correct", 0.0), res.metrics.get("is_incorrect", 0.0)
        res.metrics["accuracy_given_attempted"] = c / (c + i) if c + i > 0 else 0.0
        p, r = res.metrics["accuracy_given_attempted"], c
        res.metrics["f1"] = 2 * p * r / (p + r) if p + r > 0 else 0.0
        return res
