"""Named performance suites with regression floors.

Reference: `test/srt/nightly/single_host/suite_runner.py` (suites of launch profiles x sweep cases, each case with
floors such as `out_tps >= 865.6` for Qwen3-32B decode at concurrency 32, 4096 in / 1024 out, `:170-172`) and
`perf_case_runner.py`.  Here a case is one closed-loop run through the in-process engine (`Engine.generate`, random
token ids, random-init weights of a named architecture or a checkpoint directory): decode cases measure output
tokens per second, prefill cases (one output token) input tokens per second.  A suite fails when a case ends below
its floor.

    python -m sglang_jax_b200.test.suite_runner --suite perf-text-models-b200-1 [--tp-size 8] [--floors floors.json]
    python -m sglang_jax_b200.test.suite_runner --list

Floors are properties of a deployment: the built-in numbers are the reference's TPU v6e-4 floors scaled by nothing
(they are what a user switching over expects at least); `--floors` replaces them per case name.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import sys
import tempfile
import time

import numpy as np


@dataclasses.dataclass
class PerfCase:
    name: str
    model: str                    # key of `utils.tiny_models.ARCH_CONFIGS`, "tiny-qwen3", or a checkpoint directory
    concurrency: int
    input_len: int
    output_len: int
    num_prompts: int | None = None
    floors: dict = dataclasses.field(default_factory=dict)     # metric -> minimum
    engine_args: dict = dataclasses.field(default_factory=dict)

    @property
    def kind(self) -> str:
        return "prefill" if self.output_len <= 1 else "decode"


def perf_sweep_cases(model: str, decode_concurrencies=(16, 32), input_len=4096, output_len=1024, floors=None,
                     prefill_point=(32, 4096, 1), prefill_floors=None, engine_args=None) -> list[PerfCase]:
    """Decode points `concurrency x input_len x output_len` plus one prefill point, floors on the largest decode
    point and on the prefill point (the reference's `perf_sweep_cases`)."""
    cases = []
    for c in decode_concurrencies:
        last = c == max(decode_concurrencies)
        cases.append(PerfCase(f"{model}-decode-c{c}-i{input_len}-o{output_len}", model, c, input_len, output_len,
                              floors=dict(floors or {}) if last else {}, engine_args=dict(engine_args or {})))
    c, i, o = prefill_point
    cases.append(PerfCase(f"{model}-prefill-c{c}-i{i}", model, c, i, o, floors=dict(prefill_floors or {}),
                          engine_args=dict(engine_args or {})))
    return cases


SUITES: dict[str, list[PerfCase]] = {
    # the reference's nightly dense / MoE sweeps (its floors are for TPU v6e-4 TP4)
    "perf-text-models-b200-1": perf_sweep_cases("qwen3-32b", (16, 32), floors={"out_tps": 865.6},
                                                 prefill_floors={"in_tps": 15629.7}),
    "perf-moe-models-b200": perf_sweep_cases("qwen3-30b-a3b", (32, 64, 96), floors={"out_tps": 1534.1},
                                             prefill_floors={"in_tps": 24039.9}),
    "perf-qwen3-8b": perf_sweep_cases("qwen3-8b", (64, 256), 1024, 1024, floors={"out_tps": 5296.6},
                                      prefill_point=(256, 1024, 1), prefill_floors={"in_tps": 28299.0}),
    # seconds on a CPU: used by the test-suite and as a smoke run of the runner itself
    "smoke-cpu": perf_sweep_cases("tiny-qwen3", (2, 4), 48, 8, floors={"out_tps": 1.0}, prefill_point=(4, 48, 1),
                                  prefill_floors={"in_tps": 1.0},
                                  engine_args={"device": "cpu", "dtype": "float32", "page_size": 4}),
}


def _model_dir(model: str) -> tuple[str, dict]:
    import os
    if os.path.isdir(model):
        return model, {}
    from ..utils.tiny_models import ARCH_CONFIGS, TINY_QWEN3, write_config_only
    cfg = dict(TINY_QWEN3 if model == "tiny-qwen3" else ARCH_CONFIGS[model])
    return write_config_only(tempfile.mkdtemp(prefix="sglb_suite_"), cfg), {"load_format": "dummy"}


def run_case(case: PerfCase, engine=None, **engine_overrides) -> dict:
    """One closed-loop run; returns the metrics and `passed` / `violations` against the case's floors."""
    from ..entrypoints.engine import Engine
    own = engine is None
    if own:
        path, extra = _model_dir(case.model)
        kw = dict(model_path=path, skip_tokenizer_init=True, enable_single_process=True, log_level="error",
                  max_running_requests=max(case.concurrency, 8), disable_radix_cache=True, watchdog_timeout=0, **extra)
        kw.update(case.engine_args)
        kw.update(engine_overrides)
        engine = Engine(**kw)
    try:
        vocab = engine.scheduler.model_config.vocab_size if engine.scheduler is not None else 32000
        n = case.num_prompts or 2 * case.concurrency
        rng = np.random.RandomState(0)
        prompts = [rng.randint(5, max(vocab - 5, 6), size=case.input_len).tolist() for _ in range(n)]
        sp = {"temperature": 0.0, "max_new_tokens": case.output_len, "ignore_eos": True}
        done_in = done_out = 0
        t0 = time.perf_counter()
        # closed loop: `concurrency` requests in flight, in waves of that size
        for i in range(0, n, case.concurrency):
            outs = engine.generate(input_ids=prompts[i:i + case.concurrency], sampling_params=sp)
            done_in += sum(o["meta_info"]["prompt_tokens"] for o in outs)
            done_out += sum(o["meta_info"]["completion_tokens"] for o in outs)
        wall = time.perf_counter() - t0
    finally:
        if own:
            engine.shutdown()
    metrics = {"in_tps": done_in / wall, "out_tps": done_out / wall, "wall_s": wall, "requests": n}
    violations = {k: (metrics[k], v) for k, v in case.floors.items() if metrics.get(k, 0.0) < v}
    return {"case": case.name, "kind": case.kind, **metrics, "floors": case.floors, "passed": not violations,
            "violations": violations}


def run_suite(name: str, floors: dict | None = None, **engine_overrides) -> list[dict]:
    from ..parallel import state as ps
    results = []
    for case in SUITES[name]:
        if floors and case.name in floors:
            case = dataclasses.replace(case, floors=floors[case.name])
        ps.reset_state()
        results.append(run_case(case, **engine_overrides))
        print(json.dumps(results[-1]), flush=True)
    return results


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--suite", default=None)
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--floors", default=None, help="JSON file: {case name: {metric: minimum}}")
    ap.add_argument("--tp-size", type=int, default=None)
    ap.add_argument("--device", default=None)
    ns = ap.parse_args(argv)
    if ns.list or not ns.suite:
        for k, cases in SUITES.items():
            print(k, [c.name for c in cases])
        return 0
    floors = json.load(open(ns.floors)) if ns.floors else None
    over = {k: v for k, v in (("tp_size", ns.tp_size), ("device", ns.device)) if v is not None}
    res = run_suite(ns.suite, floors, **over)
    bad = [r for r in res if not r["passed"]]
    print(json.dumps({"suite": ns.suite, "cases": len(res), "failed": [r["case"] for r in bad]}))
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
