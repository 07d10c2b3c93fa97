"""`python -m sglang_jax_b200.profiler --url http://host:port --num-steps 5`: asks a running server
to trace the next N forward steps (reference `python/sgl_jax/profiler.py:19-68`) and stores the
server's arguments beside the trace."""

from __future__ import annotations

import argparse
import json
import os
import time

import requests


def run_profile(url: str, num_steps: int, output_dir: str | None, profile_by_stage: bool = False,
                activities: list[str] | None = None, profile_name: str | None = None,
                profile_stages: list[str] | None = None):
    output_dir = os.path.abspath(output_dir or os.environ.get("SGLANG_PROFILER_DIR", "/tmp/sglang_profile"))
    os.makedirs(output_dir, exist_ok=True)
    info = requests.get(url + "/get_server_info", timeout=30).json()
    with open(os.path.join(output_dir, "server_args.json"), "w") as f:
        json.dump({k: v for k, v in info.items() if k != "internal_states"}, f, indent=1)
    body = {"output_dir": output_dir, "num_steps": num_steps, "profile_by_stage": profile_by_stage}
    if activities:
        body["activities"] = activities
    if profile_name:
        body["profile_name"] = profile_name
    if profile_stages:
        body["profile_stages"] = profile_stages
    r = requests.post(url + "/start_profile", json=body, timeout=60)
    r.raise_for_status()
    print(f"profiling {num_steps} steps into {output_dir}")
    while requests.get(url + "/profile_status", timeout=30).json().get("status") == "profiling":
        time.sleep(1)
    return output_dir


if __name__ == "__main__":
    p = argparse.ArgumentParser()
    p.add_argument("--url", default="http://127.0.0.1:30000")
    p.add_argument("--output-dir", default=None)
    p.add_argument("--num-steps", type=int, default=5)
    p.add_argument("--profile-by-stage", action="store_true")
    p.add_argument("--profile-stages", default=None, help="comma-separated stages, e.g. prefill,decode")
    p.add_argument("--profile-name", default=None, help="file-name stem of the traces")
    p.add_argument("--cpu", action=argparse.BooleanOptionalAction, default=True, help="host activity")
    p.add_argument("--gpu", action=argparse.BooleanOptionalAction, default=True, help="device activity")
    p.add_argument("--mem", action=argparse.BooleanOptionalAction, default=False,
                   help="allocator history as a snapshot for pytorch.org/memory_viz")
    p.add_argument("--rpd", action="store_true", help="accepted for the reference's command lines (ROCm only): ignored")
    a = p.parse_args()
    acts = [n for n, on in (("CPU", a.cpu), ("GPU", a.gpu), ("MEM", a.mem)) if on]
    run_profile(a.url, a.num_steps, a.output_dir, a.profile_by_stage, acts, a.profile_name,
                a.profile_stages.split(",") if a.profile_stages else None)
