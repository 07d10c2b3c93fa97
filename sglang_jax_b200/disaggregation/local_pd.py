"""One front door over prefill and decode engines on the GPUs of one node (`--pd-disaggregation`).

The reference's in-process P/D split (`python/sgl_jax/srt/disaggregation/pathways_pd.py`,
`pathways_scheduler.py`; flags `--pd-disaggregation`, `--pd-num-prefill`, `--pd-num-decode`,
`--pd-prefill-tp-size`, `--pd-prefill-ep-size`, `--pd-{prefill,decode}-mem-fraction`,
`--pd-{prefill,decode}-max-tokens`) drives a prefill mesh and a decode mesh from one controller and moves KV between
them with a device-to-device put, so a client sees one server.  Here the same deployment is `pd_num_prefill` prefill
engines and `pd_num_decode` decode engines, each on its own slice of `device_indexes` with its own tensor-parallel
size, memory fraction and prefill budget, wired to an embedded bootstrap registry; the KV crosses NVLink through the
CUDA-IPC hand-over (or the TCP path on CPU).  `LocalPDEngine` gives them the `Engine` surface: every request gets a
bootstrap room, goes to one prefill engine (round robin) and one decode engine (fewest requests in flight) at the
same time, and the decode engine's answer is returned.
"""

from __future__ import annotations

import copy
import itertools
import logging
import secrets
import threading
from concurrent.futures import ThreadPoolExecutor

from fastapi import FastAPI, Request          # module level: the route signatures are resolved from these names
from fastapi.responses import JSONResponse

logger = logging.getLogger(__name__)


class LocalPDEngine:
    def __init__(self, server_args):
        from ..entrypoints.engine import Engine
        from ..utils.common import get_free_port
        from .bootstrap import BootstrapServer
        sa = server_args
        self.server_args = sa
        n_p, n_d = max(int(sa.pd_num_prefill), 1), max(int(sa.pd_num_decode), 1)
        tp_d = sa.tp_size
        tp_p = int(sa.pd_prefill_tp_size) or tp_d
        need = n_p * tp_p + n_d * tp_d
        devices = list(sa.device_indexes) if sa.device_indexes else list(range(need))
        if len(devices) < need:
            raise ValueError(f"--pd-disaggregation needs {need} devices ({n_p} x tp{tp_p} prefill + {n_d} x tp{tp_d} "
                             f"decode), device_indexes lists {len(devices)}")
        secret = sa.disaggregation_shared_secret or secrets.token_hex(16)
        port = sa.disaggregation_bootstrap_port if sa.disaggregation_bootstrap_url is None else None
        self.bootstrap = None
        url = sa.disaggregation_bootstrap_url
        if url is None:
            try:
                self.bootstrap = BootstrapServer(port=port, secret=secret).start()
            except Exception:          # the configured port is taken (several launchers on one host)
                self.bootstrap = BootstrapServer(port=get_free_port(), secret=secret).start()
            url = self.bootstrap.url

        def sub(mode: str, index: int, slice_):
            s = copy.copy(sa)
            s.pd_disaggregation = ""
            s.disaggregation_mode = mode
            s.disaggregation_bootstrap_url, s.disaggregation_shared_secret = url, secret
            s.disaggregation_transfer_port = s.disaggregation_side_channel_port = 0
            s.disaggregation_engine_id = f"{mode}-{index}"
            s.device_indexes = list(slice_)
            s.dp_size = 1
            s.enable_engine_loop_run_forever_daemon = True      # calls from several threads may overlap on an engine
            if mode == "prefill":
                s.tp_size = tp_p
                s.ep_size = int(sa.pd_prefill_ep_size) or (max(sa.ep_size * tp_p // tp_d, 1) if sa.ep_size > 1 else 1)
                s.mem_fraction_static = sa.pd_prefill_mem_fraction
                s.max_prefill_tokens = max(int(sa.pd_prefill_max_tokens), s.chunked_prefill_size or 0)
            else:
                s.mem_fraction_static = sa.pd_decode_mem_fraction
                if sa.max_total_tokens is None and sa.pd_decode_max_tokens and sa.device == "cpu":
                    s.max_total_tokens = int(sa.pd_decode_max_tokens)
            s.port = sa.port + 100 * (1 + index + (0 if mode == "prefill" else n_p))
            return Engine(server_args=s)

        self.prefill, self.decode = [], []
        try:
            off = 0
            for i in range(n_p):
                self.prefill.append(sub("prefill", i, devices[off:off + tp_p]))
                off += tp_p
            for i in range(n_d):
                self.decode.append(sub("decode", i, devices[off:off + tp_d]))
                off += tp_d
        except BaseException:
            self.shutdown()
            raise
        self._rooms = itertools.count(1)
        self._rr = itertools.count()
        self._inflight = [0] * n_d
        self._lock = threading.Lock()
        self._locks = {"prefill": [threading.Lock() for _ in range(n_p)], "decode": [threading.Lock() for _ in range(n_d)]}
        self._pool = ThreadPoolExecutor(max_workers=2 * max(n_p + n_d, 4))
        self.routed = {"prefill": [0] * n_p, "decode": [0] * n_d}
        self.tokenizer_manager = self.decode[0].tokenizer_manager
        logger.info("in-node PD: %d prefill (tp%d) + %d decode (tp%d) engines, registry %s", n_p, tp_p, n_d, tp_d, url)

    # ------------------------------------------------------------------ generation
    def _pick(self) -> tuple[int, int]:
        with self._lock:
            p = next(self._rr) % len(self.prefill)
            d = min(range(len(self.decode)), key=lambda i: (self._inflight[i], i))
            self._inflight[d] += 1
            self.routed["prefill"][p] += 1
            self.routed["decode"][d] += 1
        return p, d

    def _call(self, eng, lock, idx, prompts, ids, sps, rooms, kw):
        """One batched `generate` on one engine (the engines run their event loop on a thread of their own, so calls
        of concurrent `generate`s of this front door overlap)."""
        args = dict(sampling_params=[sps[i] for i in idx], bootstrap_room=[rooms[i] for i in idx], **kw)
        if ids is not None:
            args["input_ids"] = [ids[i] for i in idx]
        else:
            args["prompt"] = [prompts[i] for i in idx]
        return eng.generate(**args)

    def generate(self, prompt=None, sampling_params=None, input_ids=None, **kw):
        single = isinstance(prompt, str) or (input_ids is not None and len(input_ids) > 0
                                             and isinstance(input_ids[0], int))
        prompts = [prompt] if isinstance(prompt, str) else prompt
        ids = [input_ids] if (single and input_ids is not None) else input_ids
        n = len(ids) if ids is not None else len(prompts)
        sps = sampling_params if isinstance(sampling_params, list) else [sampling_params] * n
        kw.pop("bootstrap_room", None)
        picks = [self._pick() for _ in range(n)]
        rooms = [next(self._rooms) for _ in range(n)]
        by_p: dict[int, list[int]] = {}
        by_d: dict[int, list[int]] = {}
        for i, (p, d) in enumerate(picks):
            by_p.setdefault(p, []).append(i)
            by_d.setdefault(d, []).append(i)
        try:
            fp = [self._pool.submit(self._call, self.prefill[p], self._locks["prefill"][p], idx, prompts, ids, sps,
                                    rooms, kw) for p, idx in by_p.items()]
            fd = {d: self._pool.submit(self._call, self.decode[d], self._locks["decode"][d], idx, prompts, ids, sps,
                                       rooms, kw) for d, idx in by_d.items()}
            outs = [None] * n
            for d, idx in by_d.items():
                for i, o in zip(idx, fd[d].result()):
                    o.setdefault("meta_info", {}).update(pd_prefill_engine=picks[i][0], pd_decode_engine=d,
                                                         bootstrap_room=rooms[i])
                    outs[i] = o
            for f in fp:
                f.result()
        finally:
            with self._lock:
                for _, d in picks:
                    self._inflight[d] -= 1
        return outs[0] if single else outs

    # ------------------------------------------------------------------ fan-out controls
    def engines(self):
        return list(self.prefill) + list(self.decode)

    def flush_cache(self):
        return [e.flush_cache() for e in self.engines()]

    def get_server_info(self) -> dict:
        infos = [e.get_server_info() for e in self.engines()]
        out = dict(infos[-1])
        out["internal_states"] = [s for i in infos for s in i.get("internal_states", [])]
        out["pd_routed"] = {k: list(v) for k, v in self.routed.items()}
        return out

    def abort_request(self, rid: str = "", abort_all: bool = False):
        for e in self.engines():
            e.abort_request(rid, abort_all)

    def shutdown(self):
        from .runtime import shutdown_disaggregation
        for e in self.engines():
            sched = getattr(e, "scheduler", None)
            if sched is not None:
                try:
                    shutdown_disaggregation(sched, 1)
                except Exception:      # noqa: BLE001
                    logger.exception("PD shutdown of an engine failed")
            try:
                e.shutdown()
            except Exception:          # noqa: BLE001
                logger.exception("engine shutdown failed")
        self.prefill, self.decode = [], []
        if getattr(self, "_pool", None) is not None:
            self._pool.shutdown(wait=False)
        if self.bootstrap is not None:
            self.bootstrap.stop()
            self.bootstrap = None


def build_pd_app(engine: LocalPDEngine):
    """HTTP surface of the in-node PD front door: `/generate` (non-streaming; text or token ids, one request or a
    batch), `/health`, `/get_server_info`, `/flush_cache`, `/abort_request`.  The OpenAI routes are served by the
    per-role servers behind `launch_router`; this app is what `launch_server --pd-disaggregation` exposes."""
    import asyncio
    app = FastAPI()

    @app.get("/health")
    async def health():
        return JSONResponse({"status": "ok", "prefill": len(engine.prefill), "decode": len(engine.decode)})

    @app.get("/get_server_info")
    async def info():
        return JSONResponse(engine.get_server_info())

    @app.post("/flush_cache")
    async def flush():
        await asyncio.get_running_loop().run_in_executor(None, engine.flush_cache)
        return JSONResponse({"success": True})

    @app.post("/abort_request")
    async def abort(request: Request):
        body = await request.json()
        engine.abort_request(body.get("rid", ""), bool(body.get("abort_all", False)))
        return JSONResponse({"success": True})

    @app.post("/generate")
    async def generate(request: Request):
        body = await request.json()
        if body.get("stream"):
            return JSONResponse({"error": "streaming is served by the per-role servers behind launch_router"}, 400)
        kw = {k: body[k] for k in ("return_logprob", "logprob_start_len", "top_logprobs_num", "lora_path") if k in body}
        try:
            out = await asyncio.get_running_loop().run_in_executor(
                None, lambda: engine.generate(prompt=body.get("text"), sampling_params=body.get("sampling_params"),
                                              input_ids=body.get("input_ids"), **kw))
        except ValueError as e:
            return JSONResponse({"error": str(e)}, 400)
        return JSONResponse(out)

    return app
