"""Latency of one batch through a running server (reference `python/sgl_jax/bench_one_batch_server.py`)."""

from __future__ import annotations

import argparse
import json
import time

import numpy as np
import requests


def run_one_case(url: str, batch_size: int, input_len: int, output_len: int, vocab_size: int = 32000) -> dict:
    rng = np.random.RandomState(0)
    ids = [rng.randint(0, vocab_size, input_len).tolist() for _ in range(batch_size)]
    body = {"input_ids": ids, "stream": True,
            "sampling_params": {"temperature": 0, "max_new_tokens": output_len, "ignore_eos": True}}
    t0 = time.perf_counter()
    ttft = None
    with requests.post(url + "/generate", json=body, stream=True, timeout=3600) as r:
        for line in r.iter_lines():
            if line and line.startswith(b"data:") and not line.endswith(b"[DONE]"):
                if ttft is None:
                    ttft = time.perf_counter() - t0
    lat = time.perf_counter() - t0
    return {"batch_size": batch_size, "input_len": input_len, "output_len": output_len, "latency_s": lat,
            "ttft_s": ttft, "input_throughput": batch_size * input_len / (ttft or lat),
            "output_throughput": batch_size * output_len / max(lat - (ttft or 0), 1e-9)}


if __name__ == "__main__":
    p = argparse.ArgumentParser()
    p.add_argument("--base-url", default="http://127.0.0.1:30000")
    p.add_argument("--batch-size", type=int, nargs="+", default=[1, 16])
    p.add_argument("--input-len", type=int, nargs="+", default=[1024])
    p.add_argument("--output-len", type=int, nargs="+", default=[16])
    ns = p.parse_args()
    for bs in ns.batch_size:
        for il in ns.input_len:
            for ol in ns.output_len:
                print(json.dumps(run_one_case(ns.base_url, bs, il, ol)))
