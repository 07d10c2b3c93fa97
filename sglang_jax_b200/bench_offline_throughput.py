"""Offline throughput through the in-process `Engine` (reference `python/sgl_jax/bench_offline_throughput.py`).

    python -m sglang_jax_b200.bench_offline_throughput --model-path ... --num-prompts 256
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import time

from .bench_serving import sample_random_requests
from .server_args import ServerArgs


def throughput_test(server_args: ServerArgs, num_prompts=256, input_len=1024, output_len=128, range_ratio=1.0,
                    vocab_size=None, seed=1) -> dict:
    from .entrypoints.engine import Engine
    eng = Engine(server_args=server_args)
    try:
        vocab = vocab_size or eng.tokenizer_manager.model_config.vocab_size
        reqs = sample_random_requests(input_len, output_len, num_prompts, range_ratio, vocab, seed)
        sps = [{"temperature": 0.0, "max_new_tokens": o, "ignore_eos": True} for _, o in reqs]
        eng.generate(input_ids=[reqs[0][0]], sampling_params=[{**sps[0], "max_new_tokens": 4}])   # warm-up
        t0 = time.perf_counter()
        outs = eng.generate(input_ids=[r[0] for r in reqs], sampling_params=sps)
        dt = time.perf_counter() - t0
        n_in = sum(len(r[0]) for r in reqs)
        n_out = sum(o["meta_info"]["completion_tokens"] for o in outs)
        return {"successful_requests": len(outs), "total_latency": dt, "total_input_tokens": n_in,
                "total_output_tokens": n_out, "request_throughput": len(outs) / dt,
                "input_throughput": n_in / dt, "output_throughput": n_out / dt,
                "total_throughput": (n_in + n_out) / dt}
    finally:
        eng.shutdown()


if __name__ == "__main__":
    p = argparse.ArgumentParser()
    ServerArgs.add_cli_args(p)
    p.add_argument("--num-prompts", type=int, default=256)
    p.add_argument("--random-input-len", type=int, default=1024)
    p.add_argument("--random-output-len", type=int, default=128)
    p.add_argument("--random-range-ratio", type=float, default=1.0)
    ns = p.parse_args()
    sa = ServerArgs.from_cli_args(ns)
    print(json.dumps(throughput_test(sa, ns.num_prompts, ns.random_input_len, ns.random_output_len,
                                     ns.random_range_ratio)))
