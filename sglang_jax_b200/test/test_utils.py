"""Helpers for server-level tests and benchmarks (reference `python/sgl_jax/test/test_utils.py`:
`popen_launch_server` :278, `run_bench_serving` :524, `run_bench_one_batch` :615,
`run_bench_offline_throughput` :668)."""

from __future__ import annotations

import json
import os
import socket
import subprocess
import sys
import time

DEFAULT_TIMEOUT_FOR_SERVER_LAUNCH = 600


def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def popen_launch_server(model: str, base_url: str | None = None, timeout: float = DEFAULT_TIMEOUT_FOR_SERVER_LAUNCH,
                        other_args: list[str] | None = None, env: dict | None = None, api_key: str | None = None,
                        check_cache_miss: bool = True, stdout=None, stderr=None) -> subprocess.Popen:
    """Start `python -m sglang_jax_b200.launch_server` and wait until `/health_generate` answers.
    `check_cache_miss` turns a CUDA-graph recapture while serving into a failed request."""
    if base_url is None:
        base_url = f"http://127.0.0.1:{find_free_port()}"
    host, port = base_url.split("://", 1)[1].rsplit(":", 1)
    cmd = [sys.executable, "-m", "sglang_jax_b200.launch_server", "--model-path", model, "--host", host, "--port", port,
           *(other_args or [])]
    if api_key:
        cmd += ["--api-key", api_key]
    e = dict(os.environ, **(env or {}))
    if check_cache_miss:
        e["SGLANG_ENABLE_CACHE_MISS_CHECK"] = "1"
    proc = subprocess.Popen(cmd, env=e, stdout=stdout, stderr=stderr)
    proc.base_url = base_url
    import requests
    t0 = time.time()
    headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    while time.time() - t0 < timeout:
        if proc.poll() is not None:
            raise RuntimeError(f"server exited with code {proc.returncode} while starting")
        try:
            if requests.get(base_url + "/health_generate", headers=headers, timeout=5).status_code == 200:
                return proc
        except requests.RequestException:
            pass
        time.sleep(0.5)
    kill_process_tree(proc)
    raise TimeoutError(f"server did not become healthy within {timeout} s")


def kill_process_tree(proc: subprocess.Popen, wait: float = 10.0):
    """Stop exactly the server we started and its children."""
    try:
        import psutil
        parent = psutil.Process(proc.pid)
        procs = parent.children(recursive=True) + [parent]
        for p in procs:
            try:
                p.terminate()
            except psutil.NoSuchProcess:
                pass
        _, alive = psutil.wait_procs(procs, timeout=wait)
        for p in alive:
            try:
                p.kill()
            except psutil.NoSuchProcess:
                pass
    except ImportError:
        proc.terminate()
        try:
            proc.wait(wait)
        except subprocess.TimeoutExpired:
            proc.kill()


def _run_module(module: str, args: list[str], timeout: float = 3600) -> dict:
    out = subprocess.run([sys.executable, "-m", module, *args], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                         timeout=timeout)
    if out.returncode != 0:
        raise RuntimeError(f"{module} failed:\n{out.stderr[-2000:]}")
    for line in reversed(out.stdout.strip().splitlines()):
        try:
            return json.loads(line)
        except json.JSONDecodeError:
            continue
    return {"stdout": out.stdout}


def run_bench_serving(base_url: str, num_prompts: int = 64, random_input_len: int = 256, random_output_len: int = 64,
                      max_concurrency: int | None = None, extra: list[str] | None = None) -> dict:
    host, port = base_url.split("://", 1)[1].rsplit(":", 1)
    args = ["--host", host, "--port", port, "--dataset-name", "random", "--num-prompts", str(num_prompts),
            "--random-input-len", str(random_input_len), "--random-output-len", str(random_output_len),
            "--random-range-ratio", "1"]
    if max_concurrency:
        args += ["--max-concurrency", str(max_concurrency)]
    return _run_module("sglang_jax_b200.bench_serving", args + (extra or []))


def run_bench_one_batch(model: str, other_args: list[str] | None = None) -> dict:
    return _run_module("sglang_jax_b200.bench_one_batch", ["--model-path", model, *(other_args or [])])


def run_bench_offline_throughput(model: str, other_args: list[str] | None = None) -> dict:
    return _run_module("sglang_jax_b200.bench_offline_throughput", ["--model-path", model, *(other_args or [])])
