"""Latency of one static batch without a server or scheduler (reference `python/sgl_jax/bench_one_batch.py`):
prefill of `batch_size x input_len` then `output_len` decode steps straight on the `ModelRunner`.

    python -m sglang_jax_b200.bench_one_batch --model-path ... --batch-size 16 --input-len 1024 --output-len 32
"""

from __future__ import annotations

import argparse
import json
import time

import numpy as np
import torch

from .server_args import ServerArgs


def run_one_batch(server_args: ServerArgs, batch_size: int, input_len: int, output_len: int,
                  log_decode_step: int = 0) -> dict:
    from .configs.model_config import ModelConfig
    from .managers.schedule_batch import ForwardMode, ModelWorkerBatch, ModelWorkerSamplingInfo
    from .model_executor.model_runner import ModelRunner
    from .parallel import state as ps
    if not ps.get_state().initialized:
        ps.init_distributed(0, 1, server_args.device)
    runner = ModelRunner(ModelConfig.from_server_args(server_args), server_args)
    pool, P = runner.req_to_token_pool, runner.page_size
    rng = np.random.RandomState(0)
    vocab = runner.model_config.vocab_size
    B = batch_size
    per_req = (input_len + output_len + P - 1) // P * P
    base = np.arange(B, dtype=np.int64) * per_req + P

    def greedy(n):
        return ModelWorkerSamplingInfo(np.ones(n, np.float32), np.ones(n, np.float32), np.ones(n, np.int32),
                                       np.zeros(n, np.float32), None, True, False, False, False)

    def sync():
        if runner.device.type == "cuda":
            torch.cuda.synchronize()

    locs = np.concatenate([b + np.arange(input_len) for b in base]).astype(np.int32)
    for b in range(B):
        pool.write(b, 0, base[b] + np.arange(input_len))
    rows, pos, ids = pool.take_page_deltas()
    batch = ModelWorkerBatch(
        bid=0, forward_mode=ForwardMode.EXTEND, input_ids=rng.randint(0, vocab, B * input_len).astype(np.int32),
        req_pool_indices=np.arange(B, dtype=np.int32), seq_lens=np.full(B, input_len, np.int32), out_cache_loc=locs,
        positions=np.tile(np.arange(input_len, dtype=np.int32), B), extend_prefix_lens=np.zeros(B, np.int32),
        extend_seq_lens=np.full(B, input_len, np.int32), extend_logprob_start_lens=np.zeros(B, np.int32),
        page_delta_rows=rows, page_delta_pos=pos, page_delta_ids=ids, sampling_info=greedy(B))
    sync()
    t0 = time.perf_counter()
    _, tok, _ = runner.forward(batch)
    sync()
    prefill_s = time.perf_counter() - t0
    decode = []
    tok_np = tok.cpu().numpy()
    for step in range(output_len):
        n = input_len + step
        for b in range(B):
            pool.set_one(b, n, int(base[b] + n))
        rows, pos, ids = pool.take_page_deltas()
        db = ModelWorkerBatch(bid=step + 1, forward_mode=ForwardMode.DECODE, input_ids=tok_np.astype(np.int32),
                              req_pool_indices=np.arange(B, dtype=np.int32), seq_lens=np.full(B, n + 1, np.int32),
                              out_cache_loc=(base + n).astype(np.int32), positions=np.full(B, n, np.int32),
                              page_delta_rows=rows, page_delta_pos=pos, page_delta_ids=ids, sampling_info=greedy(B))
        sync()
        t0 = time.perf_counter()
        _, tok, _ = runner.forward(db)
        tok_np = tok.cpu().numpy()
        decode.append(time.perf_counter() - t0)
        if log_decode_step and (step + 1) % log_decode_step == 0:
            print(f"decode step {step + 1}: {decode[-1] * 1e3:.2f} ms, {B / decode[-1]:.1f} tok/s", flush=True)
    med = float(np.median(decode)) if decode else 0.0
    return {"batch_size": B, "input_len": input_len, "output_len": output_len, "prefill_latency_s": prefill_s,
            "prefill_throughput": B * input_len / prefill_s, "median_decode_latency_s": med,
            "decode_throughput": B / med if med else 0.0,
            "total_latency_s": prefill_s + sum(decode)}


def correctness_test(server_args: ServerArgs, cut_len: int = 4, output_len: int = 8, prompts=None) -> dict:
    """`--correctness-test` (reference `bench_one_batch.py` `correctness_test`): every prompt is generated twice,
    prefilled in one piece and prefilled as `cut_len` tokens followed by the rest (the second part extends a cached
    prefix); both must give the same greedy continuation, which is printed."""
    from .entrypoints.engine import Engine
    from .parallel import state as ps
    prompts = prompts or [list(range(11, 11 + 3 * cut_len)), list(range(40, 40 + 2 * cut_len + 1)),
                          [7, 3, 9] * (cut_len + 1)]
    sp = {"temperature": 0.0, "max_new_tokens": output_len, "ignore_eos": True}
    P = server_args.page_size
    cut = max(cut_len // P, 1) * P                      # a cached prefix is whole pages
    outs = {}
    for name in ("whole", "split"):
        ps.reset_state()
        eng = Engine(server_args=server_args)
        try:
            if name == "split":
                eng.generate(input_ids=[p[:cut] for p in prompts if len(p) > cut],
                             sampling_params={**sp, "max_new_tokens": 1})
            res = eng.generate(input_ids=prompts, sampling_params=sp)
            outs[name] = [o["output_ids"] for o in res]
            outs[name + "_cached"] = [o["meta_info"].get("cached_tokens", 0) for o in res]
        finally:
            eng.shutdown()
    for i, (a, b) in enumerate(zip(outs["whole"], outs["split"])):
        print(f"prompt {i}: whole {a}\n          split {b} (cached {outs['split_cached'][i]})")
    ok = outs["whole"] == outs["split"]
    print("correctness test", "passed" if ok else "FAILED")
    return {"passed": ok, **outs}


def main(argv=None) -> list[dict]:
    p = argparse.ArgumentParser()
    ServerArgs.add_cli_args(p)
    p.add_argument("--batch-size", type=int, nargs="+", default=[1])
    p.add_argument("--input-len", type=int, nargs="+", default=[1024])
    p.add_argument("--output-len", type=int, nargs="+", default=[16])
    p.add_argument("--run-name", default="default")
    p.add_argument("--result-filename", default=None, help="append one JSON line per configuration")
    p.add_argument("--log-decode-step", type=int, default=0, help="print the latency of every n-th decode step")
    p.add_argument("--correctness-test", action="store_true")
    p.add_argument("--cut-len", type=int, default=4)
    p.add_argument("--prompt-filename", default=None, help="correctness test: a JSON list of token-id prompts")
    p.add_argument("--profile", action="store_true", help="a torch profiler trace per configuration")
    p.add_argument("--profile-filename-prefix", default="profile")
    ns = p.parse_args(argv)
    sa = ServerArgs.from_cli_args(ns)
    if ns.correctness_test:
        prompts = None
        if ns.prompt_filename:
            with open(ns.prompt_filename) as f:
                prompts = json.load(f)
        return [correctness_test(sa, ns.cut_len, ns.output_len[0], prompts)]
    out = []
    for bs in ns.batch_size:
        for il in ns.input_len:
            for ol in ns.output_len:
                if ns.profile:
                    from torch.profiler import ProfilerActivity, profile
                    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
                    with profile(activities=acts) as prof:
                        rec = run_one_batch(sa, bs, il, ol, ns.log_decode_step)
                    name = f"{ns.profile_filename_prefix}_batch{bs}_input{il}_output{ol}.trace.json"
                    prof.export_chrome_trace(name)
                    rec["profile"] = name
                else:
                    rec = run_one_batch(sa, bs, il, ol, ns.log_decode_step)
                rec["run_name"] = ns.run_name
                print(json.dumps(rec))
                out.append(rec)
                if ns.result_filename:
                    with open(ns.result_filename, "a") as f:
                        f.write(json.dumps(rec) + "\n")
    return out


if __name__ == "__main__":
    main()
