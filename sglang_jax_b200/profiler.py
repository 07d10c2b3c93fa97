"""`python -m sglang_jax_b200.profiler --url http://host:port --num-steps 5`: asks a running server
to trace the next N forward steps (reference `python/sgl_jax/profiler.py:19-68`) and stores the
server's arguments beside the trace."""

from __future__ import annotations

import argparse
import json
import os
import time

import requests


def run_profile(url: str, num_steps: int, output_dir: str | None, profile_by_stage: bool = False):
    output_dir = os.path.abspath(output_dir or os.environ.get("SGLANG_PROFILER_DIR", "/tmp/sglang_profile"))
    os.makedirs(output_dir, exist_ok=True)
    info = requests.get(url + "/get_server_info", timeout=30).json()
    with open(os.path.join(output_dir, "server_args.json"), "w") as f:
        json.dump({k: v for k, v in info.items() if k != "internal_states"}, f, indent=1)
    r = requests.post(url + "/start_profile", json={"output_dir": output_dir, "num_steps": num_steps,
                                                    "profile_by_stage": profile_by_stage}, timeout=60)
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
    a = p.parse_args()
    run_profile(a.url, a.num_steps, a.output_dir, a.profile_by_stage)
