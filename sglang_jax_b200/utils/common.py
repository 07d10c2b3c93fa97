"""Process / logging helpers (reference `python/sgl_jax/srt/utils/common_utils.py`)."""

from __future__ import annotations

import ctypes
import json
import logging
import logging.config
import os
import signal
import socket
import sys
import threading
import time


def configure_logger(server_args, prefix: str = ""):
    """`SGLANG_LOGGING_CONFIG_PATH` may point to a JSON dictConfig that replaces the default."""
    path = os.environ.get("SGLANG_LOGGING_CONFIG_PATH")
    if path:
        with open(path) as f:
            logging.config.dictConfig(json.load(f))
        return
    fmt = f"[%(asctime)s{prefix}] %(message)s"
    logging.basicConfig(level=getattr(logging, str(server_args.log_level).upper(), logging.INFO), format=fmt,
                        datefmt="%Y-%m-%d %H:%M:%S", force=True)


def kill_itself_when_parent_died():
    """Linux: deliver SIGKILL to this process when its parent exits."""
    if sys.platform == "linux":
        PR_SET_PDEATHSIG = 1
        try:
            ctypes.CDLL("libc.so.6").prctl(PR_SET_PDEATHSIG, signal.SIGKILL)
        except Exception:
            pass


def kill_process_tree(parent_pid: int | None = None, include_parent: bool = True, skip_pid: int | None = None):
    import psutil
    if parent_pid is None:
        parent_pid = os.getpid()
        include_parent = False
    try:
        parent = psutil.Process(parent_pid)
    except psutil.NoSuchProcess:
        return
    for child in parent.children(recursive=True):
        if child.pid == skip_pid:
            continue
        try:
            child.kill()
        except psutil.NoSuchProcess:
            pass
    if include_parent:
        try:
            parent.kill()
        except psutil.NoSuchProcess:
            pass


def get_free_port() -> int:
    """A port that is free now and is unlikely to be taken before the caller binds it: ports below the kernel's
    ephemeral range are tried first (an ephemeral port handed back by `bind(0)` can be grabbed by any outgoing
    connection of this machine between this call and the caller's own bind)."""
    import random
    for _ in range(64):
        port = random.randint(20000, 31999)
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            try:
                s.bind(("127.0.0.1", port))
                return port
            except OSError:
                continue
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def is_port_available(port: int) -> bool:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        try:
            s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            s.bind(("", port))
            return True
        except OSError:
            return False


def get_bool_env_var(name: str, default: str = "false") -> bool:
    return os.environ.get(name, default).lower() in ("1", "true", "yes")


def set_prometheus_multiproc_dir():
    import tempfile
    d = tempfile.mkdtemp(prefix="sglb200_prom_")
    os.environ["PROMETHEUS_MULTIPROC_DIR"] = d
    return d


def add_prometheus_middleware(app):
    from prometheus_client import CollectorRegistry, make_asgi_app, multiprocess
    registry = CollectorRegistry()
    if os.environ.get("PROMETHEUS_MULTIPROC_DIR"):
        multiprocess.MultiProcessCollector(registry)
        app.mount("/metrics", make_asgi_app(registry=registry))
    else:
        app.mount("/metrics", make_asgi_app())


def add_api_key_middleware(app, api_key: str):
    from starlette.responses import JSONResponse

    @app.middleware("http")
    async def authentication(request, call_next):
        if request.method == "OPTIONS" or request.url.path.startswith(("/health", "/metrics", "/ping")):
            return await call_next(request)
        if request.headers.get("Authorization") != "Bearer " + api_key:
            return JSONResponse(content={"error": "Unauthorized"}, status_code=401)
        return await call_next(request)


def launch_dummy_health_check_server(host: str, port: int):
    """Non-zero nodes answer /health so orchestrators see them alive (reference :404)."""
    import uvicorn
    from fastapi import FastAPI, Response
    app = FastAPI()

    @app.get("/health")
    async def health():
        return Response(status_code=200)

    @app.get("/health_generate")
    async def health_generate():
        return Response(status_code=200)

    uvicorn.run(app, host=host, port=port, log_level="warning")


def pyspy_dump_schedulers():
    import faulthandler
    faulthandler.dump_traceback()


class TimeStats:
    """Wall-clock checkpoints of one request through the pipeline."""

    def __init__(self):
        self.t = {"created": time.perf_counter()}

    def mark(self, name: str):
        self.t[name] = time.perf_counter()

    def span(self, a: str, b: str) -> float | None:
        if a in self.t and b in self.t:
            return self.t[b] - self.t[a]
        return None
