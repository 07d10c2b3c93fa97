#!/usr/bin/env python
"""Headline serving benchmark: steady-state output tokens/s of a named model (default Qwen3-32B,
bf16, random-init, synthetic random-token requests with input lengths uniform in [512, 2048],
256 output tokens, concurrency 128) on N GPUs of one node, tensor parallel over all N.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

What is timed.  The engine is first brought to the steady state of a closed loop at `concurrency`
(untimed): every row of the running batch is decoding, the requests' remaining output lengths are
spread evenly over one replacement cycle (request i of the fill has `ceil((i+1) * out / concurrency)`
tokens left and its prompt is longer by the tokens it "already generated"), and a finished request is
replaced by a fresh one at once.  From then on the schedule is periodic: decode steps of the full
batch interleaved with the prefill of each replacement.  A "step" is one scheduler iteration that
launches a forward batch.  After W warm-up steps exactly K steps are timed with CUDA events on every
rank (barrier + synchronize on both sides, max over ranks); `value` = output tokens those K steps
produced / that time.  The schedule depends only on the seed, never on timing, so the same K steps
(and the same `timed_tokens`) are measured at every N.

`e2e` is the same metric through the public API: `Engine.generate(input_ids=[...])` for
`--e2e-requests` requests (default 2 x concurrency; the named config's 2048 with `--e2e-requests 2048`),
wall clock, including every step's host->device copy of the batch integers from pinned memory and the
device->host read of the sampled tokens.  `latency` is a streamed closed loop through
`Engine.async_generate(stream=True)` at the same concurrency: p50 TTFT (first chunk) and p50 ITL (gaps
between chunks), the definitions of the reference's serving benchmark
(`python/sgl_jax/bench_serving.py:1942-2117`).

`--impl nccl` runs the same engine with the fused NVLink kernels off (library collectives): the A/B
arm of this repo.  `--impl reference` drives the unmodified reference from `baseline/_ref` through its
own `Engine`; it needs JAX, and prints the `unavailable` line when JAX cannot be imported.
"""

from __future__ import annotations

import argparse
import asyncio
import json
import math
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# request shapes of the named configurations: (input min, input max, output, concurrency)
MODEL_SHAPES = {
    "qwen3-32b": (512, 2048, 256, 128),
    "qwen3-32b-tp8-shard": (512, 2048, 256, 128),
    "llama3-8b": (1024, 1024, 512, 64),
    "qwen3-8b": (1024, 1024, 1024, 64),
    "qwen3-30b-a3b": (1024, 1024, 512, 256),
    "deepseek-v3": (2048, 2048, 512, 128),
    "tiny-qwen3": (16, 64, 16, 8),
}

# Nearest published figure of the reference per model (output tok/s; all on TPU, other request shapes):
# context for `vs_baseline`, not a like-for-like target.
PUBLISHED = {
    "qwen3-32b": (1977.45, "TPU v6e-4 TP4, 1024/1024 c=64 (docs/cookbook/autoregressive/Qwen/Qwen3.md:471)"),
    "qwen3-8b": (5296.60, "TPU v6e-4 TP4, 1024/1024 c=64 (docs/cookbook/autoregressive/Qwen/Qwen3.md:462)"),
    "llama3-8b": (1448.91, "TPU v6e-4 TP4, 512/512 c=16 (docs/cookbook/autoregressive/Llama/Llama3.1.md:166)"),
    "qwen3-30b-a3b": (6179.45, "TPU v7x-4 TP8 EP8, 1024/1024 c=128 (docs/cookbook/autoregressive/Qwen/Qwen3-MoE.md:378)"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--warmup", type=int, default=6)
    ap.add_argument("--impl", default="ours", choices=["ours", "nccl", "reference"])
    ap.add_argument("--fused-max-tokens", type=int, default=None,
                    help="A/B arm: forwards of at most this many rows use the fused NVLink residual dataflow "
                         "(1000000 = every forward; default: the engine's own default)")
    ap.add_argument("--model", default="qwen3-32b")
    ap.add_argument("--concurrency", type=int, default=None)
    ap.add_argument("--input-len-min", type=int, default=None)
    ap.add_argument("--input-len-max", type=int, default=None)
    ap.add_argument("--output-len", type=int, default=None)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--chunked-prefill-size", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (result marked invalid)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-latency", action="store_true")
    ap.add_argument("--e2e-requests", type=int, default=None, help="requests of the end-to-end pass (default 2 x concurrency)")
    ap.add_argument("--latency-requests", type=int, default=None, help="requests of the streamed pass (default 2 x concurrency)")
    ap.add_argument("--shared-prefix", action="store_true",
                    help="end-to-end pass on the shared-prefix variant: groups of 128 requests sharing a 1536-token "
                         "prefix plus a 128-token unique suffix")
    ap.add_argument("--quantization", default=None)
    ap.add_argument("--moe-backend", default=None)
    ap.add_argument("--enable-mixed-chunk", action="store_true",
                    help="let prefill steps carry the running batch's decode tokens (the server flag of the same name)")
    ap.add_argument("--disable-cuda-graph", action="store_true")
    ap.add_argument("--disable-fused-comm", action="store_true")
    ap.add_argument("--disable-overlap", action="store_true")
    ap.add_argument("--device", default=None)
    ap.add_argument("--log-level", default="error")
    ap.add_argument("--hang-timeout", type=float, default=float(os.environ.get("SGLB_BENCH_HANG_TIMEOUT", "300")),
                    help="seconds without progress after which every rank dumps its stacks and exits")
    a = ap.parse_args()
    lo, hi, out, conc = MODEL_SHAPES.get(a.model, MODEL_SHAPES["qwen3-32b"])
    a.input_len_min = lo if a.input_len_min is None else a.input_len_min
    a.input_len_max = hi if a.input_len_max is None else a.input_len_max
    a.output_len = out if a.output_len is None else a.output_len
    a.concurrency = conc if a.concurrency is None else a.concurrency
    return a


def metric_name(model: str) -> str:
    pretty = {"qwen3-32b": "Qwen3-32B", "llama3-8b": "Llama-3-8B", "qwen3-8b": "Qwen3-8B",
              "qwen3-30b-a3b": "Qwen3-30B-A3B", "deepseek-v3": "DeepSeek-V3"}.get(model, model)
    return f"output tok/s (device-timed, max over ranks) {pretty}"


# ------------------------------------------------------------------------------------ reference arm
def reference_arm(args):
    """The unmodified reference (`baseline/_ref`, installed with `pip --target`) through its own public
    API: `sgl_jax.srt.entrypoints.engine.Engine(**server_args)` and `Engine.generate(input_ids=...)`
    (reference `python/sgl_jax/srt/entrypoints/engine.py:71,:150`), same model shape, request shapes,
    concurrency and dtype.  The reference is single-controller (one process drives every device), so only
    rank 0 of a multi-rank launch runs it; the others exit at once."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    try:
        import jax  # noqa: F401
    except Exception as e:
        print(json.dumps({"impl": "reference",
                          "unavailable": f"reference needs JAX ({type(e).__name__}: {e}); jax/jaxlib/flax are not "
                                         f"installed and not in the offline wheelhouse"}))
        return 0
    try:
        import numpy as np
        from sgl_jax.srt.entrypoints.engine import Engine as RefEngine

        # architecture tables only (plain dicts + a config.json writer), loaded by path so that nothing of this
        # repo's engine, models or kernels is imported on the reference's path
        import importlib.util
        spec = importlib.util.spec_from_file_location(
            "_arch_tables", os.path.join(ROOT, "sglang_jax_b200", "utils", "tiny_models.py"))
        tables = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(tables)
        ARCH_CONFIGS, write_config_only = tables.ARCH_CONFIGS, tables.write_config_only

        n_dev = len([d for d in jax.devices() if d.platform in ("gpu", "cuda")])
        if n_dev < args.gpus:
            raise RuntimeError(f"JAX sees {n_dev} CUDA devices, {args.gpus} requested")
        cfg = dict(ARCH_CONFIGS[args.model])
        max_len = args.input_len_max + args.output_len + 64
        cfg["max_position_embeddings"] = max(4096, max_len)
        model_dir = write_config_only(os.path.join(tempfile.gettempdir(), f"sglref_{args.model}"), cfg)
        # `dummy` is the reference's own weight generator for a config-only directory
        eng = RefEngine(model_path=model_dir, load_format="dummy", tp_size=args.gpus, device="cuda",
                        dtype="bfloat16", page_size=args.page_size, chunked_prefill_size=args.chunked_prefill_size,
                        max_running_requests=args.concurrency, context_length=cfg["max_position_embeddings"],
                        skip_tokenizer_init=True, attention_backend="native", mem_fraction_static=0.85,
                        log_level="error", random_seed=0)
        rng = np.random.RandomState(0)
        vocab = cfg["vocab_size"]
        n_req = args.e2e_requests or 2 * args.concurrency
        prompts = [rng.randint(0, vocab, size=int(rng.randint(args.input_len_min, args.input_len_max + 1))).tolist()
                   for _ in range(n_req)]
        sp = {"max_new_tokens": args.output_len, "temperature": 0.0, "ignore_eos": True}
        eng.generate(input_ids=prompts[: min(8, n_req)], sampling_params=dict(sp, max_new_tokens=8))   # compile
        t0 = time.perf_counter()
        outs = eng.generate(input_ids=prompts, sampling_params=sp)
        t1 = time.perf_counter()
        n_tok = sum(len(o["output_ids"]) for o in outs)
        val = n_tok / (t1 - t0)
        print(json.dumps({
            "metric": metric_name(args.model), "value": round(val, 2), "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "impl": "reference",
            "data": "synthetic random token ids, the reference's dummy weights of the named architecture",
            "timing": "wall clock around Engine.generate (the reference exposes no per-step device events)",
            "config": {"model": args.model, "global_batch": args.concurrency,
                       "seq_len": f"in U[{args.input_len_min},{args.input_len_max}] out {args.output_len}",
                       "parallelism": f"tp{args.gpus}", "requests": n_req},
            "e2e": {"value": val, "unit": "tok/s", "requests": n_req, "wall_s": round(t1 - t0, 3)}}), flush=True)
        eng.shutdown()
    except Exception as e:
        print(json.dumps({"impl": "reference", "unavailable": f"reference did not run: {type(e).__name__}: {e}"[:400]}))
    return 0


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(prefix="clocks_", suffix=".csv")
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    mx.append(float(p[2]))
                except ValueError:
                    continue
                for n, v in zip(names, p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _leave(world: int):
    """End a rank of a multi-rank run without tearing the communicators down: with captured CUDA graphs that
    hold library collectives still alive, the teardown can wait forever for a peer that has already gone."""
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        os._exit(0)


def percentile(xs, q):
    if not xs:
        return None
    xs = sorted(xs)
    k = (len(xs) - 1) * q
    lo, hi = int(math.floor(k)), int(math.ceil(k))
    return xs[lo] + (xs[hi] - xs[lo]) * (k - lo)


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl == "nccl":
        args.disable_fused_comm = True
    if args.fused_max_tokens is not None:
        os.environ["SGLB_FUSED_MAX_TOKENS"] = str(args.fused_max_tokens)

    import numpy as np
    import torch

    from sglang_jax_b200.managers.io_struct import TokenizedGenerateReqInput
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.sampling.sampling_params import SamplingParams
    from sglang_jax_b200.server_args import ServerArgs
    from sglang_jax_b200.utils.tiny_models import ARCH_CONFIGS, TINY_QWEN3, write_config_only

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (launch with torch.distributed.run); "
                             f"WORLD_SIZE={world}")
    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    # A stuck collective must not burn the whole time limit: without progress for `hang_timeout`
    # seconds the process prints every thread's stack and exits non-zero.
    import faulthandler

    def arm():
        if args.hang_timeout and args.hang_timeout > 0:
            faulthandler.dump_traceback_later(args.hang_timeout, exit=True)

    arm()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    moe_model = args.model in ("qwen3-30b-a3b", "deepseek-v3")
    ps.init_distributed(rank, world, device, 1, world if moe_model else 1, local_rank=local_rank,
                        init_method="env://" if world > 1 else None)

    cfg = dict(TINY_QWEN3 if args.model == "tiny-qwen3" else ARCH_CONFIGS[args.model])
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    L, C = args.output_len, args.concurrency
    max_len = args.input_len_max + 2 * L + 64
    cfg["max_position_embeddings"] = max(4096, max_len)
    model_dir = write_config_only(os.path.join(tempfile.gettempdir(), f"sglb200_{args.model}_{rank}"), cfg)
    extra = {}
    if args.quantization:
        extra["quantization"] = args.quantization
    if args.moe_backend:
        extra["moe_backend"] = args.moe_backend
    if args.enable_mixed_chunk:
        extra["enable_mixed_chunk"] = True
    sa = ServerArgs(
        model_path=model_dir, load_format="dummy", tp_size=world, ep_size=world if moe_model else 1, device=device,
        dtype="bfloat16" if device == "cuda" else "float32",
        page_size=args.page_size, chunked_prefill_size=args.chunked_prefill_size,
        max_prefill_tokens=max(16384, args.chunked_prefill_size), max_running_requests=C,
        context_length=cfg["max_position_embeddings"], skip_tokenizer_init=True, enable_single_process=True,
        disable_cuda_graph=args.disable_cuda_graph, disable_fused_comm=args.disable_fused_comm,
        disable_overlap_schedule=args.disable_overlap, cuda_graph_max_bs=C,
        disable_radix_cache=False, log_level=args.log_level, watchdog_timeout=0, decode_log_interval=1 << 30,
        mem_fraction_static=0.9, **extra)

    if rank != 0:
        from sglang_jax_b200.managers.tp_worker import run_tp_follower
        run_tp_follower(sa, on_message=arm)
        faulthandler.cancel_dump_traceback_later()
        _leave(world)
        return 0

    from sglang_jax_b200 import Engine
    from sglang_jax_b200.ops import native

    t_init = time.time()
    engine = Engine(server_args=sa)
    sched = engine.scheduler
    worker = sched.tp_worker
    init_s = time.time() - t_init

    rng = np.random.RandomState(0)
    vocab = cfg["vocab_size"]

    def new_request(i: int, remaining: int | None = None) -> TokenizedGenerateReqInput:
        n = int(rng.randint(args.input_len_min, args.input_len_max + 1))
        out = L
        if remaining is not None:
            # a request of the steady state that has `remaining` tokens to go: the tokens it already
            # produced are part of its context
            n += L - remaining
            out = remaining
        ids = rng.randint(0, vocab, size=n).tolist()
        return TokenizedGenerateReqInput(
            rid=f"bench-{i}", input_ids=ids,
            sampling_params=SamplingParams(max_new_tokens=out, temperature=0.0, ignore_eos=True))

    # ---------------- phase 1: K device-timed steps of the steady-state closed loop
    W, K = args.warmup, args.steps
    state = {"steps": 0, "submitted": 0, "phase": "fill", "d2h": 0, "launch0": 0, "replay0": 0,
             "done": threading.Event(), "replaced": 0, "fill_steps": 0}
    seen: dict[str, int] = {}          # request id -> output tokens produced so far
    runner = getattr(worker, "model_runner", None)
    clocks = ClockSampler(local_rank)

    finished: set = set()              # ids of requests seen finished

    def top_up(s):
        # requests in flight = submitted (some may still sit in the scheduler's input queue) - finished
        live = state["submitted"] - len(finished)
        while live < C and state["phase"] != "done":
            i = state["submitted"]
            s._recv_q.put(new_request(i, None if i >= C else -(-(i + 1) * L // C)))
            state["submitted"] += 1
            if i >= C:
                state["replaced"] += 1
            live += 1

    def total_tokens() -> int:
        return sum(seen.values())

    def hook(s, batch):
        if state["phase"] == "done":
            return
        if batch is None:
            top_up(s)
            return
        for r in batch.reqs:
            seen[r.rid] = len(r.output_ids)
            if r.finished():
                finished.add(r.rid)
        top_up(s)
        arm()
        if state["phase"] == "fill":
            state["fill_steps"] += 1
            # steady state: every row decodes, and the first replacement has been prefilled and merged
            if state["replaced"] >= 1 and batch.forward_mode.is_decode() and len(batch.reqs) >= C - 1 \
                    and not s.waiting_queue and s.chunked_req is None:
                state["phase"] = "warmup"
            if state["phase"] == "fill":
                return
        state["steps"] += 1
        now = time.perf_counter()
        this_kind = "decode" if batch.forward_mode.is_decode() else "prefill"
        if state["phase"] == "timed":
            # With overlap scheduling this hook runs after batch i was launched and batch i-1's result was waited
            # for, so the interval that ends here is the device time of batch i-1: it is booked to that batch's kind.
            kind = state.get("prev_kind", this_kind) if s.enable_overlap else this_kind
            state[kind + "_s"] = state.get(kind + "_s", 0.0) + now - state["last_t"]
            state[kind + "_n"] = state.get(kind + "_n", 0) + 1
            if not batch.forward_mode.is_decode():
                state["prefill_tok"] = state.get("prefill_tok", 0) + int(sum(batch.extend_lens))
                state["prefill_batches"] = state.get("prefill_batches", 0) + 1
            state["d2h"] += 4 * len(batch.reqs)
        state["prev_kind"] = this_kind
        state["last_t"] = now
        if state["steps"] == W + 1 and state["phase"] == "warmup":
            # the steady state's first step counts as warm-up step 0; W more have run since
            if device == "cuda":
                torch.cuda.synchronize()
            state["launch0"] = native.launch_count
            state["replay0"] = runner.graph_replays if runner is not None else 0
            state["h2d0"] = getattr(runner, "h2d_bytes_total", 0) if runner is not None else 0
            clocks.start()
            worker.mark("t0")
            state["tok0"] = total_tokens()
            state["phase"] = "timed"
            state["wall0"] = state["last_t"] = time.perf_counter()
        elif state["steps"] == W + 1 + K and state["phase"] == "timed":
            worker.mark("t1")
            if device == "cuda":
                torch.cuda.synchronize()
            state["wall1"] = time.perf_counter()
            state["tok1"] = total_tokens()
            state["launches"] = native.launch_count - state["launch0"]
            state["replays"] = (runner.graph_replays if runner is not None else 0) - state["replay0"]
            state["h2d1"] = getattr(runner, "h2d_bytes_total", 0) if runner is not None else 0
            state["phase"] = "done"
            state["done"].set()

    sched.step_hooks.append(hook)      # the scheduler thread's idle iterations call it: requests are only ever
    state["done"].wait()               # submitted from that one thread
    arm()
    clock_info = clocks.stop()
    ms = worker.elapsed_ms_max_over_ranks("t0", "t1")
    sched.step_hooks.remove(hook)
    engine.abort_request(abort_all=True)
    # let the scheduler retire the aborted requests
    for _ in range(400):
        time.sleep(0.05)
        if not sched.running_batch.reqs and not sched.waiting_queue and sched.chunked_req is None \
                and not sched.result_queue:
            break
    timed_tokens = state["tok1"] - state["tok0"]
    value = timed_tokens / (ms / 1e3)

    # kernels launched inside a replayed CUDA graph are counted once at capture time
    kpg = 0
    gr = getattr(runner, "cuda_graph_runner", None) if runner is not None else None
    if gr is not None and gr.graphs:
        kpg = getattr(gr, "kernels_per_graph", 0)
    gpu_launches = state.get("launches", 0) + state.get("replays", 0) * kpg

    arm()
    sp = {"max_new_tokens": L, "temperature": 0.0, "ignore_eos": True}

    def make_prompts(n_req: int):
        if args.shared_prefix:
            out, group = [], None
            for i in range(n_req):
                if i % 128 == 0:
                    group = rng.randint(0, vocab, size=1536).tolist()
                out.append(group + rng.randint(0, vocab, size=128).tolist())
            return out
        return [rng.randint(0, vocab, size=int(rng.randint(args.input_len_min, args.input_len_max + 1))).tolist()
                for _ in range(n_req)]

    # ---------------- phase 2: the same workload through the public API, wall clock
    e2e = None
    if not args.no_e2e:
        n_req = args.e2e_requests or 2 * C
        prompts = make_prompts(n_req)
        h2d0 = getattr(runner, "h2d_bytes_total", 0) if runner is not None else 0
        f0 = sched.forward_ct
        if device == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = engine.generate(input_ids=prompts, sampling_params=sp)
        t1 = time.perf_counter()
        n_tok = sum(len(o["output_ids"]) for o in outs)
        steps2 = max(sched.forward_ct - f0, 1)
        h2d = ((getattr(runner, "h2d_bytes_total", 0) if runner is not None else 0) - h2d0) // steps2
        e2e = {"value": n_tok / (t1 - t0), "unit": "tok/s", "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(4 * n_tok // steps2), "requests": n_req, "wall_s": round(t1 - t0, 3),
               "shared_prefix": bool(args.shared_prefix)}
        if args.shared_prefix:
            e2e["cached_tokens"] = int(sum(o["meta_info"].get("cached_tokens", 0) for o in outs))
        arm()

    # ---------------- phase 3: streamed closed loop at `concurrency`: p50 TTFT / ITL
    latency = None
    if not args.no_latency:
        n_req = args.latency_requests or 2 * C
        prompts = make_prompts(n_req)
        ttft, itl, lat = [], [], []

        async def one(ids, sem):
            async with sem:
                st = time.perf_counter()
                last, n_seen = st, 0
                gen = await engine.async_generate(input_ids=ids, sampling_params=sp, stream=True)
                async for chunk in gen:
                    now = time.perf_counter()
                    n = len(chunk["output_ids"])
                    if n > n_seen:
                        if n_seen == 0:
                            ttft.append(now - st)
                        else:
                            itl.extend([(now - last) / (n - n_seen)] * (n - n_seen))
                        n_seen, last = n, now
                lat.append(time.perf_counter() - st)
                arm()

        async def run_all():
            sem = asyncio.Semaphore(C)
            await asyncio.gather(*[one(p, sem) for p in prompts])

        t0 = time.perf_counter()
        engine.loop.run_until_complete(run_all())
        t1 = time.perf_counter()
        latency = {"p50_ttft_ms": round(1e3 * percentile(ttft, 0.5), 2), "p50_itl_ms": round(1e3 * percentile(itl, 0.5), 3),
                   "p99_ttft_ms": round(1e3 * percentile(ttft, 0.99), 2), "p99_itl_ms": round(1e3 * percentile(itl, 0.99), 3),
                   "mean_tpot_ms": round(1e3 * sum((a - b) / max(L - 1, 1) for a, b in zip(lat, ttft)) / max(len(lat), 1), 3),
                   "requests": n_req, "concurrency": C, "output_tok_s": round(n_req * L / (t1 - t0), 2),
                   "definition": "streamed Engine.async_generate, closed loop; TTFT = first chunk, ITL = gaps between chunks"}

    native_status = "ok"
    try:
        if device == "cuda":
            native.check_status()
    except Exception as e:
        native_status = str(e)

    st = ps.get_state()
    parallelism = f"tp{world}" + (f"+ep{world}" if moe_model and world > 1 else "")
    pub = PUBLISHED.get(args.model)
    dn, pn = state.get("decode_n", 0), state.get("prefill_n", 0)
    out = {
        "metric": metric_name(args.model), "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": round(value / pub[0], 4) if pub else None,
        "baseline_note": (f"{pub[0]} tok/s published by the reference on {pub[1]}: other hardware and request shape, "
                          f"context only") if pub else "the reference publishes no number for this model",
        "dtype": ("bf16" if device == "cuda" else "fp32") + (f"+{args.quantization}" if args.quantization else ""),
        "data": "synthetic random token ids, random-init weights (normal 0.02) of the named architecture",
        "impl": args.impl,
        "config": {"model": args.model, "global_batch": C, "seq_len": f"in U[{args.input_len_min},"
                   f"{args.input_len_max}] out {L}", "parallelism": parallelism,
                   "page_size": args.page_size, "chunked_prefill_size": args.chunked_prefill_size,
                   "l2": "inputs larger than L2: every step streams the full per-GPU weight shard "
                         f"({runner.weight_bytes / 2**30:.1f} GiB) plus KV" if runner is not None else "n/a",
                   "window": "steady-state closed loop (staggered fill, periodic decode/prefill mix)",
                   "cuda_graph": gr is not None, "fused_comm": st.fused_comm is not None,
                   "fused_tokens": ([runner.fused_min_tokens, runner.fused_max_tokens]
                                    if st.fused_comm is not None and runner is not None else None),
                   "tp_dataflow": (None if world == 1 else
                                   "fused NVLink kernels for forwards inside fused_tokens, NCCL all-reduce + add-RMSNorm "
                                   "otherwise" if (st.fused_comm is not None and runner is not None
                                                   and runner.fused_max_tokens >= runner.fused_min_tokens)
                                   else "NCCL all-reduce + add-RMSNorm"),
                   "mixed_chunk": bool(sa.enable_mixed_chunk),
                   "overlap_schedule": sched.enable_overlap, "layers": cfg["num_hidden_layers"]},
        "clocks": clock_info, "e2e": e2e, "latency": latency,
        "p50_ttft_ms": latency["p50_ttft_ms"] if latency else None,
        "p50_itl_ms": latency["p50_itl_ms"] if latency else None,
        "gpu_launches": int(gpu_launches),
        "timed_tokens": int(timed_tokens), "init_s": round(init_s, 1), "fill_steps": state["fill_steps"],
        "kernel_status": native_status,
        "wall_ms_per_step": round((state["wall1"] - state["wall0"]) * 1e3 / K, 4),
        "timed_h2d_bytes_per_step": int((state.get("h2d1", 0) - state.get("h2d0", 0)) // max(K, 1)),
        "step_breakdown": {"decode": {"steps": dn, "host_ms_per_step": round(1e3 * state.get("decode_s", 0.0) / max(dn, 1), 3)},
                           "prefill": {"steps": pn, "host_ms_per_step": round(1e3 * state.get("prefill_s", 0.0) / max(pn, 1), 3),
                                       "tokens_per_step": round(state.get("prefill_tok", 0)
                                                                / max(state.get("prefill_batches", 0), 1), 1)}},
    }
    if args.layers:
        out["invalid"] = "debug run with fewer layers than the named model"
    faulthandler.cancel_dump_traceback_later()
    print(json.dumps(out), flush=True)
    engine.shutdown()
    _leave(world)
    return 0


if __name__ == "__main__":
    sys.exit(main())
