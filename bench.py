#!/usr/bin/env python
"""Headline serving benchmark: output tokens/s of Qwen3-32B (bf16, random-init, synthetic
random-token requests with input lengths uniform in [512, 2048], 256 output tokens,
concurrency 128) on N GPUs of one node, tensor parallel over all N.

    python bench.py --gpus 1 --steps 600 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 600 --warmup 8

A "step" is one scheduler iteration that launches a forward batch (a prefill chunk or a
decode step of the running batch) in steady-state continuous batching.  After W warm-up
steps exactly K steps are timed with CUDA events on every rank (max over ranks);
`value` = output tokens produced by those K steps / that time.  `e2e` is the same metric
through the public API: `Engine.generate(input_ids=[...], sampling_params=...)` for 2 x
concurrency requests, wall clock, including every step's host->device copy of the batch
integers from pinned memory and the device->host read of the sampled tokens.

`--impl reference` would run the unmodified reference from `baseline/_ref`; it needs JAX,
which is neither installed nor in the offline wheelhouse, so it prints the `unavailable` line.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "output tok/s (device-timed, max over ranks) Qwen3-32B"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=600)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-32b")
    ap.add_argument("--concurrency", type=int, default=128)
    ap.add_argument("--input-len-min", type=int, default=512)
    ap.add_argument("--input-len-max", type=int, default=2048)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--chunked-prefill-size", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (result marked invalid)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--disable-cuda-graph", action="store_true")
    ap.add_argument("--disable-fused-comm", action="store_true")
    ap.add_argument("--disable-overlap", action="store_true")
    ap.add_argument("--device", default=None)
    ap.add_argument("--log-level", default="error")
    ap.add_argument("--hang-timeout", type=float, default=float(os.environ.get("SGLB_BENCH_HANG_TIMEOUT", "300")),
                    help="seconds without progress after which every rank dumps its stacks and exits")
    return ap.parse_args()


def reference_arm(args):
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    try:
        import jax  # noqa: F401
        import sgl_jax  # noqa: F401
    except Exception as e:
        print(json.dumps({"impl": "reference",
                          "unavailable": f"reference needs JAX ({type(e).__name__}: {e}); jax/jaxlib/flax are not "
                                         f"installed and not in the offline wheelhouse"}))
        return 0
    print(json.dumps({"impl": "reference", "unavailable": "reference GPU path not wired on this box"}))
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
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=self.f,
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


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import numpy as np
    import torch

    from sglang_jax_b200.managers.io_struct import TokenizedGenerateReqInput
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.sampling.sampling_params import SamplingParams
    from sglang_jax_b200.server_args import ServerArgs
    from sglang_jax_b200.utils.tiny_models import ARCH_CONFIGS, write_config_only

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
    ps.init_distributed(rank, world, device, local_rank=local_rank, init_method="env://" if world > 1 else None)

    cfg = dict(ARCH_CONFIGS[args.model])
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    max_len = args.input_len_max + args.output_len + 64
    cfg["max_position_embeddings"] = max(4096, max_len)
    model_dir = write_config_only(os.path.join(tempfile.gettempdir(), f"sglb200_{args.model}_{rank}"), cfg)
    sa = ServerArgs(
        model_path=model_dir, load_format="dummy", tp_size=world, device=device,
        dtype="bfloat16" if device == "cuda" else "float32",
        page_size=args.page_size, chunked_prefill_size=args.chunked_prefill_size,
        max_prefill_tokens=max(16384, args.chunked_prefill_size), max_running_requests=args.concurrency,
        context_length=cfg["max_position_embeddings"], skip_tokenizer_init=True, enable_single_process=True,
        disable_cuda_graph=args.disable_cuda_graph, disable_fused_comm=args.disable_fused_comm,
        disable_overlap_schedule=args.disable_overlap, cuda_graph_max_bs=args.concurrency,
        disable_radix_cache=False, log_level=args.log_level, watchdog_timeout=0, decode_log_interval=1 << 30,
        mem_fraction_static=0.9)

    if rank != 0:
        from sglang_jax_b200.managers.tp_worker import run_tp_follower
        run_tp_follower(sa, on_message=arm)
        faulthandler.cancel_dump_traceback_later()
        ps.destroy()
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

    def new_request(i: int) -> TokenizedGenerateReqInput:
        n = int(rng.randint(args.input_len_min, args.input_len_max + 1))
        ids = rng.randint(0, vocab, size=n).tolist()
        return TokenizedGenerateReqInput(
            rid=f"bench-{i}", input_ids=ids,
            sampling_params=SamplingParams(max_new_tokens=args.output_len, temperature=0.0, ignore_eos=True))

    # ---------------- phase 1: K device-timed steps under a closed loop at `concurrency`
    W, K = args.warmup, args.steps
    state = {"steps": 0, "tokens": 0, "submitted": 0, "phase": "warmup", "h2d": 0, "d2h": 0,
             "launch0": 0, "replay0": 0, "done": threading.Event(), "kernels_per_graph": 0}
    runner = getattr(worker, "model_runner", None)
    clocks = ClockSampler(local_rank)

    def top_up(s):
        live = len(s.running_batch.reqs) + len(s.waiting_queue) + (1 if s.chunked_req is not None else 0)
        if s.last_batch is not None and s.last_batch.forward_mode is not None and s.last_batch.forward_mode.is_extend():
            live += sum(1 for r in s.last_batch.reqs if r not in s.running_batch.reqs and r is not s.chunked_req
                        and not r.finished())
        while live < args.concurrency and state["phase"] != "done":
            s._recv_q.put(new_request(state["submitted"]))
            state["submitted"] += 1
            live += 1

    def hook(s, batch):
        if state["phase"] == "done":
            return
        top_up(s)
        if batch is None:
            return
        state["steps"] += 1
        arm()
        now = time.perf_counter()
        if state["phase"] == "timed" and "last_t" in state:
            kind = "decode" if batch.forward_mode.is_decode() else "prefill"
            state.setdefault(kind + "_s", 0.0)
            state.setdefault(kind + "_n", 0)
            state[kind + "_s"] += now - state["last_t"]
            state[kind + "_n"] += 1
        state["last_t"] = now
        if state["phase"] == "timed":
            if batch.forward_mode.is_decode():
                state["tokens"] += len(batch.reqs)
                state["d2h"] += 4 * len(batch.reqs)
            else:
                n_out = sum(1 for r in batch.reqs if r is not batch.chunked_req)
                state["tokens"] += n_out
                state["d2h"] += 4 * len(batch.reqs)
        if state["steps"] == W and state["phase"] == "warmup":
            if device == "cuda":
                torch.cuda.synchronize()
            state["launch0"] = native.launch_count
            state["replay0"] = runner.graph_replays if runner is not None else 0
            clocks.start()
            worker.mark("t0")
            state["phase"] = "timed"
            state["wall0"] = time.perf_counter()
        elif state["steps"] == W + K and state["phase"] == "timed":
            worker.mark("t1")
            if device == "cuda":
                torch.cuda.synchronize()
            state["wall1"] = time.perf_counter()
            state["launches"] = native.launch_count - state["launch0"]
            state["replays"] = (runner.graph_replays if runner is not None else 0) - state["replay0"]
            state["phase"] = "done"
            state["done"].set()

    sched.step_hooks.append(hook)
    top_up(sched)
    state["done"].wait()
    arm()
    clock_info = clocks.stop()
    ms = worker.elapsed_ms_max_over_ranks("t0", "t1")
    sched.step_hooks.remove(hook)
    engine.abort_request(abort_all=True)
    # let the scheduler retire the aborted requests
    for _ in range(200):
        time.sleep(0.05)
        if not sched.running_batch.reqs and not sched.waiting_queue and sched.chunked_req is None \
                and not sched.result_queue:
            break
    value = state["tokens"] / (ms / 1e3)

    # kernels launched inside a replayed CUDA graph are counted once at capture time
    kpg = 0
    gr = getattr(runner, "cuda_graph_runner", None) if runner is not None else None
    if gr is not None and gr.graphs:
        kpg = getattr(gr, "kernels_per_graph", 0)
    gpu_launches = state.get("launches", 0) + state.get("replays", 0) * kpg

    arm()
    # ---------------- phase 2: the same workload through the public API, wall clock
    e2e = None
    if not args.no_e2e:
        n_req = 2 * args.concurrency
        prompts = [rng.randint(0, vocab, size=int(rng.randint(args.input_len_min, args.input_len_max + 1))).tolist()
                   for _ in range(n_req)]
        h2d0 = getattr(runner, "h2d_bytes_total", 0) if runner is not None else 0
        f0 = sched.forward_ct
        if device == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = engine.generate(input_ids=prompts, sampling_params={"max_new_tokens": args.output_len,
                                                                     "temperature": 0.0, "ignore_eos": True})
        t1 = time.perf_counter()
        n_tok = sum(len(o["output_ids"]) for o in outs)
        steps2 = max(sched.forward_ct - f0, 1)
        h2d = ((getattr(runner, "h2d_bytes_total", 0) if runner is not None else 0) - h2d0) // steps2
        e2e = {"value": n_tok / (t1 - t0), "unit": "tok/s", "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(4 * n_tok // steps2), "requests": n_req, "wall_s": round(t1 - t0, 3)}

    native_status = "ok"
    try:
        if device == "cuda":
            native.check_status()
    except Exception as e:
        native_status = str(e)

    out = {
        "metric": METRIC, "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if device == "cuda" else "fp32",
        "data": "synthetic random token ids, random-init weights (normal 0.02) of the named architecture",
        "impl": "ours",
        "config": {"model": args.model, "global_batch": args.concurrency, "seq_len": f"in U[{args.input_len_min},"
                   f"{args.input_len_max}] out {args.output_len}", "parallelism": f"tp{world}",
                   "page_size": args.page_size, "chunked_prefill_size": args.chunked_prefill_size,
                   "l2": "inputs larger than L2: every step streams the full per-GPU weight shard "
                         f"({runner.weight_bytes / 2**30:.1f} GiB) plus KV" if runner is not None else "n/a",
                   "cuda_graph": gr is not None, "fused_comm": ps.get_state().fused_comm is not None,
                   "overlap_schedule": sched.enable_overlap, "layers": cfg["num_hidden_layers"]},
        "clocks": clock_info, "e2e": e2e, "gpu_launches": int(gpu_launches),
        "timed_tokens": state["tokens"], "init_s": round(init_s, 1), "kernel_status": native_status,
        "wall_ms_per_step": round((state["wall1"] - state["wall0"]) * 1e3 / K, 4),
        "step_breakdown": {k: {"steps": state.get(k + "_n", 0),
                               "host_ms_per_step": round(1e3 * state.get(k + "_s", 0.0) / max(state.get(k + "_n", 0), 1), 3)}
                           for k in ("prefill", "decode")},
    }
    if args.layers:
        out["invalid"] = "debug run with fewer layers than the named model"
    faulthandler.cancel_dump_traceback_later()
    print(json.dumps(out), flush=True)
    engine.shutdown()
    ps.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
