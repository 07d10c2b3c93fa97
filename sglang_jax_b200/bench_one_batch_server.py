"""Latency of one batch through a running server (reference `python/sgl_jax/bench_one_batch_server.py`).

    python -m sglang_jax_b200.bench_one_batch_server --base-url http://127.0.0.1:30000 --batch-size 1 16 64 \
        --input-len 1024 --output-len 16 --show-report --result-filename one_batch.jsonl

Every (batch size, input length, output length) is one streamed request batch: TTFT is the time to the first chunk,
the rest of the latency is decoding.  `--input-len-step-percentage` shortens the prompts of a batch step by step (a
batch of unequal lengths), `--api-type openai` goes through `/v1/completions`, `--profile` brackets a case with the
server's `/start_profile` / `/stop_profile`, `--show-report` prints a table at the end.
"""

from __future__ import annotations

import argparse
import json
import time

import numpy as np
import requests


def run_one_case(url: str, batch_size: int, input_len: int, output_len: int, vocab_size: int = 32000,
                 temperature: float = 0.0, return_logprob: bool = False, stream_interval: int = 1,
                 input_len_step_percentage: float = 0.0, api_type: str = "native", run_name: str = "default",
                 model: str = "default") -> dict:
    rng = np.random.RandomState(0)
    lens = [max(int(input_len * (1.0 - input_len_step_percentage * i / max(batch_size, 1))), 1)
            for i in range(batch_size)]
    ids = [rng.randint(0, vocab_size, n).tolist() for n in lens]
    if api_type == "openai":
        path = "/v1/completions"
        body = {"model": model, "prompt": ids, "max_tokens": output_len, "temperature": temperature, "stream": True,
                "ignore_eos": True}
    else:
        path = "/generate"
        body = {"input_ids": ids, "stream": True, "return_logprob": return_logprob,
                "sampling_params": {"temperature": temperature, "max_new_tokens": output_len, "ignore_eos": True}}
    t0 = time.perf_counter()
    ttft = None
    chunks = 0
    with requests.post(url + path, json=body, stream=True, timeout=3600) as r:
        r.raise_for_status()
        for line in r.iter_lines():
            if line and line.startswith(b"data:") and not line.endswith(b"[DONE]"):
                chunks += 1
                if ttft is None and chunks >= max(stream_interval, 1):
                    ttft = time.perf_counter() - t0
    lat = time.perf_counter() - t0
    n_in = sum(lens)
    return {"run_name": run_name, "batch_size": batch_size, "input_len": input_len, "output_len": output_len,
            "latency_s": lat, "ttft_s": ttft, "input_throughput": n_in / (ttft or lat),
            "output_throughput": batch_size * output_len / max(lat - (ttft or 0), 1e-9),
            "overall_throughput": (n_in + batch_size * output_len) / lat}


def report(rows: list[dict]) -> str:
    head = f"{'batch':>6} {'input':>7} {'output':>7} {'latency s':>10} {'ttft s':>8} {'in tok/s':>10} {'out tok/s':>10}"
    lines = [head, "-" * len(head)]
    for r in rows:
        lines.append(f"{r['batch_size']:>6} {r['input_len']:>7} {r['output_len']:>7} {r['latency_s']:>10.3f} "
                     f"{(r['ttft_s'] or 0):>8.3f} {r['input_throughput']:>10.1f} {r['output_throughput']:>10.1f}")
    return "\n".join(lines)


def main(argv=None) -> list[dict]:
    p = argparse.ArgumentParser()
    p.add_argument("--base-url", default="http://127.0.0.1:30000")
    p.add_argument("--batch-size", type=int, nargs="+", default=[1, 16])
    p.add_argument("--input-len", type=int, nargs="+", default=[1024])
    p.add_argument("--output-len", type=int, nargs="+", default=[16])
    p.add_argument("--vocab-size", type=int, default=32000)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--return-logprob", action="store_true")
    p.add_argument("--client-stream-interval", type=int, default=1, help="chunks to wait for before the TTFT stamp")
    p.add_argument("--input-len-step-percentage", type=float, default=0.0)
    p.add_argument("--api-type", default="native", choices=["native", "openai"])
    p.add_argument("--model", default="default")
    p.add_argument("--run-name", default="default")
    p.add_argument("--result-filename", default=None)
    p.add_argument("--skip-warmup", action="store_true")
    p.add_argument("--profile", action="store_true")
    p.add_argument("--profile-by-stage", action="store_true", help="one profile for the prefill and one for decode")
    p.add_argument("--show-report", action="store_true")
    ns = p.parse_args(argv)
    kw = dict(vocab_size=ns.vocab_size, temperature=ns.temperature, return_logprob=ns.return_logprob,
              stream_interval=ns.client_stream_interval, input_len_step_percentage=ns.input_len_step_percentage,
              api_type=ns.api_type, run_name=ns.run_name, model=ns.model)
    if not ns.skip_warmup:
        run_one_case(ns.base_url, 1, min(ns.input_len[0], 64), 4, **kw)
    rows = []
    for bs in ns.batch_size:
        for il in ns.input_len:
            for ol in ns.output_len:
                if ns.profile:
                    body = {"num_steps": ol + 2}
                    if ns.profile_by_stage:
                        body["profile_by_stage"] = True
                    requests.post(ns.base_url + "/start_profile", json=body, timeout=60)
                rec = run_one_case(ns.base_url, bs, il, ol, **kw)
                if ns.profile:
                    requests.post(ns.base_url + "/stop_profile", timeout=60)
                print(json.dumps(rec))
                rows.append(rec)
                if ns.result_filename:
                    with open(ns.result_filename, "a") as f:
                        f.write(json.dumps(rec) + "\n")
    if ns.show_report:
        print(report(rows))
    return rows


if __name__ == "__main__":
    main()
