"""Offline throughput through the in-process `Engine` (reference `python/sgl_jax/bench_offline_throughput.py`).

    python -m sglang_jax_b200.bench_offline_throughput --model-path ... --num-prompts 256
    python -m sglang_jax_b200.bench_offline_throughput --model-path ... --dataset-name sharegpt --dataset-path sg.json

Datasets are the serving client's (`random`, `generated-shared-prefix`, `sharegpt`, `custom`); text prompts need the
engine's tokenizer, token-id prompts do not.  One warm-up batch runs first unless `--skip-warmup`; `--profile` brackets
the timed batch with the engine's profiler; `--result-filename` appends the record as a JSON line.
"""

from __future__ import annotations

import argparse
import json
import time

from .bench_serving import (_Lengths, sample_custom_requests, sample_generated_shared_prefix_requests,
                            sample_random_requests, sample_sharegpt_requests)
from .server_args import ServerArgs


def build_requests(ns, vocab_size: int) -> list:
    if ns.dataset_name == "random":
        return sample_random_requests(ns.random_input_len, ns.random_output_len, ns.num_prompts, ns.random_range_ratio,
                                      vocab_size, ns.seed)
    if ns.dataset_name == "generated-shared-prefix":
        return sample_generated_shared_prefix_requests(ns.gsp_num_groups, ns.gsp_prompts_per_group,
                                                       ns.gsp_system_prompt_len, ns.gsp_question_len,
                                                       ns.gsp_output_len, vocab_size, ns.seed)
    if not ns.dataset_path:
        raise SystemExit(f"dataset {ns.dataset_name} reads a local file: pass --dataset-path")
    lengths = _Lengths(None)
    if ns.dataset_name == "sharegpt":
        return sample_sharegpt_requests(ns.dataset_path, ns.num_prompts, lengths, ns.sharegpt_output_len,
                                        ns.sharegpt_context_len, ns.seed)
    if ns.dataset_name == "custom":
        return sample_custom_requests(ns.dataset_path, ns.num_prompts, lengths, ns.sharegpt_output_len, ns.seed)
    raise SystemExit(f"unknown dataset {ns.dataset_name}")


def throughput_test(server_args: ServerArgs, num_prompts=256, input_len=1024, output_len=128, range_ratio=1.0,
                    vocab_size=None, seed=1, ns=None) -> dict:
    """`ns`: the parsed command line (dataset and run options); without it a random dataset of the given shape."""
    from .entrypoints.engine import Engine
    eng = Engine(server_args=server_args)
    try:
        vocab = vocab_size or eng.tokenizer_manager.model_config.vocab_size
        if ns is None:
            ns = argparse.Namespace(dataset_name="random", random_input_len=input_len, random_output_len=output_len,
                                    num_prompts=num_prompts, random_range_ratio=range_ratio, seed=seed,
                                    skip_warmup=False, disable_ignore_eos=False, extra_request_body=None,
                                    prompt_suffix="", profile=False, apply_chat_template=False)
        reqs = build_requests(ns, vocab)
        extra = json.loads(ns.extra_request_body) if ns.extra_request_body else {}
        sps = [{"temperature": 0.0, "max_new_tokens": r[1], "ignore_eos": not ns.disable_ignore_eos, **extra}
               for r in reqs]
        prompts = [r[0] for r in reqs]
        text = isinstance(prompts[0], str)
        if text:
            if ns.apply_chat_template:
                tok = eng.tokenizer_manager.tokenizer
                prompts = [tok.apply_chat_template([{"role": "user", "content": p}], tokenize=False,
                                                   add_generation_prompt=True) for p in prompts]
            prompts = [p + ns.prompt_suffix for p in prompts]
        call = (lambda ps, sp: eng.generate(prompt=ps, sampling_params=sp)) if text else \
            (lambda ps, sp: eng.generate(input_ids=ps, sampling_params=sp))
        if not ns.skip_warmup:
            call(prompts[:1], [{**sps[0], "max_new_tokens": 4}])
        if ns.profile:
            eng.start_profile()
        t0 = time.perf_counter()
        outs = call(prompts, sps)
        dt = time.perf_counter() - t0
        if ns.profile:
            eng.stop_profile()
        n_in = sum(o["meta_info"].get("prompt_tokens", 0) for o in outs) or sum(len(p) for p in prompts)
        n_out = sum(o["meta_info"]["completion_tokens"] for o in outs)
        return {"backend": "engine", "dataset_name": ns.dataset_name, "successful_requests": len(outs),
                "total_latency": dt, "total_input_tokens": n_in, "total_output_tokens": n_out,
                "request_throughput": len(outs) / dt, "input_throughput": n_in / dt, "output_throughput": n_out / dt,
                "total_throughput": (n_in + n_out) / dt}
    finally:
        eng.shutdown()


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser()
    ServerArgs.add_cli_args(p)
    p.add_argument("--backend", default="engine", choices=["engine"])
    p.add_argument("--dataset-name", default="random", choices=["random", "generated-shared-prefix", "sharegpt", "custom"])
    p.add_argument("--dataset-path", default=None)
    p.add_argument("--num-prompts", type=int, default=256)
    p.add_argument("--random-input-len", type=int, default=1024)
    p.add_argument("--random-output-len", type=int, default=128)
    p.add_argument("--random-range-ratio", type=float, default=1.0)
    p.add_argument("--sharegpt-output-len", type=int, default=None)
    p.add_argument("--sharegpt-context-len", type=int, default=None)
    p.add_argument("--gsp-num-groups", type=int, default=64)
    p.add_argument("--gsp-prompts-per-group", type=int, default=16)
    p.add_argument("--gsp-system-prompt-len", type=int, default=2048)
    p.add_argument("--gsp-question-len", type=int, default=128)
    p.add_argument("--gsp-output-len", type=int, default=256)
    p.add_argument("--seed", type=int, default=1)
    p.add_argument("--disable-ignore-eos", action="store_true")
    p.add_argument("--extra-request-body", default=None, help="JSON merged into every request's sampling parameters")
    p.add_argument("--apply-chat-template", action="store_true")
    p.add_argument("--prompt-suffix", default="")
    p.add_argument("--skip-warmup", action="store_true")
    p.add_argument("--profile", action="store_true")
    p.add_argument("--result-filename", default=None)
    p.add_argument("--do-not-exit", action="store_true", help="keep the process alive after the run (for profilers)")
    return p


def main(argv=None) -> dict:
    ns = build_parser().parse_args(argv)
    sa = ServerArgs.from_cli_args(ns)
    res = throughput_test(sa, ns=ns)
    print(json.dumps(res))
    if ns.result_filename:
        with open(ns.result_filename, "a") as f:
            f.write(json.dumps(res) + "\n")
    if ns.do_not_exit:
        while True:
            time.sleep(5)
    return res


if __name__ == "__main__":
    main()
