"""`python -m sglang_jax_b200.test.run_eval --eval-name mmlu --data-path mmlu.csv --base-url http://...`
(reference `test/srt/run_eval.py`).  Datasets are read from local files; nothing is downloaded."""

from __future__ import annotations

import argparse
import json
import time

from .eval.simple_eval_common import ChatCompletionSampler, make_report


def build_eval(name: str, data_path: str, num_examples: int | None, num_threads: int, num_shots: int = 5):
    if name == "mmlu":
        from .eval.simple_eval_mmlu import MMLUEval
        return MMLUEval(data_path, num_examples, num_threads)
    if name in ("gsm8k", "mgsm"):
        from .eval.simple_eval_gsm8k import GSM8KEval
        return GSM8KEval(data_path, num_examples, num_shots, num_threads)
    from .eval import simple_eval_more as more
    if name == "math":
        return more.MathEval(data_path, num_examples, num_threads)
    if name in ("aime", "aime25", "aime26"):
        return more.AIMEEval(data_path, num_examples, num_threads)
    if name == "gpqa":
        return more.GPQAEval(data_path, num_examples, num_threads)
    if name == "humaneval":
        return more.HumanEvalEval(data_path, num_examples, min(num_threads, 16))
    if name == "mgsm_multilingual":
        return more.MGSMEval(data_path, None, num_examples, num_threads)
    raise ValueError(f"unknown eval {name!r} (mmlu, gsm8k, mgsm, math, aime, gpqa, humaneval, mgsm_multilingual; "
                     f"csimpleqa needs a grader: build `CSimpleQAEval` directly)")


def run_eval(args) -> dict:
    base = args.base_url or f"http://{args.host}:{args.port}"
    sampler = ChatCompletionSampler(base, args.model or "default", args.temperature, args.max_tokens, api_key=args.api_key)
    ev = build_eval(args.eval_name, args.data_path, args.num_examples, args.num_threads, args.num_shots)
    t0 = time.time()
    res = ev(sampler)
    out = {"eval": args.eval_name, "score": res.score, "latency_s": round(time.time() - t0, 3), **res.metrics}
    print(make_report(res))
    if args.output:
        with open(args.output, "w") as f:
            json.dump(out, f, indent=2)
    print(json.dumps(out))
    return out


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--base-url")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=30000)
    p.add_argument("--model")
    p.add_argument("--api-key")
    p.add_argument("--eval-name", default="mmlu")
    p.add_argument("--data-path", required=True)
    p.add_argument("--num-examples", type=int)
    p.add_argument("--num-threads", type=int, default=32)
    p.add_argument("--num-shots", type=int, default=5)
    p.add_argument("--max-tokens", type=int, default=2048)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--output")
    return run_eval(p.parse_args(argv))


if __name__ == "__main__":
    main()
