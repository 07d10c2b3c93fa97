"""Single-entry router for PD disaggregation (reference
`python/sgl_jax/srt/disaggregation/mini_lb.py`, `mini_lb_helpers.py`).

For every request the router picks a prefill and a decode engine, draws a `bootstrap_room`
(the transfer id both sides share), sends the request to both, and relays the decode engine's
answer (streaming included).  The prefill engine's transfer address travels to the decode
engine in `bootstrap_host` / `bootstrap_port`; it comes from the bootstrap registry."""

from __future__ import annotations

import asyncio
import contextlib
import itertools
import json
import logging
import random
import time

import aiohttp
from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, StreamingResponse

from . import pd_auth
from .bootstrap import BootstrapClient
from .router_args import RouterArgs

logger = logging.getLogger(__name__)


class PrefillEndpoint:
    def __init__(self, http_url: str, transfer_addr: str | None = None, engine_id: str | None = None):
        self.http_url = http_url.rstrip("/")
        self.transfer_addr = transfer_addr
        self.engine_id = engine_id
        self.inflight = 0


def new_room() -> int:
    return random.getrandbits(62)


class MiniLoadBalancer:
    def __init__(self, args: RouterArgs):
        self.args = args
        self.decode_urls = [u.rstrip("/") for u in args.decode_urls]
        self.prefills: list[PrefillEndpoint] = [PrefillEndpoint(u) for u in args.prefill_urls]
        self.decode_inflight = {u: 0 for u in self.decode_urls}
        self._rr_p = itertools.count()
        self._rr_d = itertools.count()
        self._registry = BootstrapClient(args.bootstrap_url, pd_auth.resolve_secret(args.shared_secret)) \
            if args.bootstrap_url else None
        self._last_refresh = 0.0
        self.routed = 0

    # ------------------------------------------------------------------ membership
    def refresh_prefills(self, force: bool = False):
        if self._registry is None:
            return
        if not force and time.time() - self._last_refresh < self.args.health_check_interval:
            return
        try:
            table = self._registry.prefills()
        except Exception as e:  # noqa: BLE001
            logger.warning("router: registry unreachable: %s", e)
            return
        known = {p.engine_id: p for p in self.prefills if p.engine_id}
        fresh = []
        for e in table["prefills"]:
            if int(e.get("tp_rank", 0)) != 0:
                continue
            p = known.get(e["engine_id"]) or PrefillEndpoint(e["http_url"], e["transfer_addr"], e["engine_id"])
            p.http_url, p.transfer_addr = e["http_url"].rstrip("/"), e["transfer_addr"]
            fresh.append(p)
        static = [p for p in self.prefills if not p.engine_id]
        self.prefills = static + fresh
        self._last_refresh = time.time()

    def pick(self) -> tuple[PrefillEndpoint, str]:
        self.refresh_prefills()
        if not self.prefills:
            self.refresh_prefills(force=True)
        if not self.prefills or not self.decode_urls:
            raise RuntimeError("router has no live prefill/decode pair")
        pol = self.args.policy
        if pol == "random":
            return random.choice(self.prefills), random.choice(self.decode_urls)
        if pol == "shortest_queue":
            return (min(self.prefills, key=lambda p: p.inflight),
                    min(self.decode_urls, key=lambda u: self.decode_inflight[u]))
        return (self.prefills[next(self._rr_p) % len(self.prefills)],
                self.decode_urls[next(self._rr_d) % len(self.decode_urls)])

    # ------------------------------------------------------------------ request path
    def _augment(self, body: dict, p: PrefillEndpoint, room: int) -> tuple[dict, dict]:
        n = None
        for k in ("text", "input_ids", "prompt"):
            v = body.get(k)
            if isinstance(v, list) and v and isinstance(v[0], (list, str)) and k != "prompt":
                n = len(v)
            elif isinstance(v, list) and v and isinstance(v[0], list):
                n = len(v)
        rooms = [room + i for i in range(n)] if n else room
        pre = dict(body, bootstrap_room=rooms, stream=False)
        dec = dict(body, bootstrap_room=rooms)
        if p.transfer_addr:
            host, port = p.transfer_addr.rsplit(":", 1)
            host = self.args.prefill_bootstrap_host or host
            dec["bootstrap_host"] = [host] * n if n else host
            dec["bootstrap_port"] = [int(port)] * n if n else int(port)
        return pre, dec

    def _gate(self):
        """`--max-concurrent-requests`: one semaphore for the router (created on the serving loop, on first use)."""
        n = int(getattr(self.args, "max_concurrent_requests", 0) or 0)
        if n <= 0:
            return contextlib.nullcontext()
        if getattr(self, "_sem", None) is None:
            self._sem = asyncio.Semaphore(n)
        return self._sem

    async def forward(self, path: str, body: dict):
        """Returns `(status, json)` for non-streaming bodies."""
        async with self._gate():
            return await self._forward(path, body)

    async def _forward(self, path: str, body: dict):
        p, d = self.pick()
        pre, dec = self._augment(body, p, new_room())
        p.inflight += 1
        self.decode_inflight[d] += 1
        self.routed += 1
        timeout = aiohttp.ClientTimeout(total=self.args.request_timeout)
        try:
            async with aiohttp.ClientSession(timeout=timeout) as sess:
                t_pre = asyncio.create_task(sess.post(p.http_url + path, json=pre))
                t_dec = asyncio.create_task(sess.post(d + path, json=dec))
                r_pre, r_dec = await asyncio.gather(t_pre, t_dec)
                if r_pre.status != 200:
                    return r_pre.status, await r_pre.json(content_type=None)
                return r_dec.status, await r_dec.json(content_type=None)
        finally:
            p.inflight -= 1
            self.decode_inflight[d] -= 1

    async def forward_stream(self, path: str, body: dict):
        """Async generator of raw SSE chunks from the decode engine."""
        async with self._gate():
            async for chunk in self._forward_stream(path, body):
                yield chunk

    async def _forward_stream(self, path: str, body: dict):
        p, d = self.pick()
        pre, dec = self._augment(body, p, new_room())
        p.inflight += 1
        self.decode_inflight[d] += 1
        self.routed += 1
        timeout = aiohttp.ClientTimeout(total=self.args.request_timeout)
        try:
            async with aiohttp.ClientSession(timeout=timeout) as sess:
                t_pre = asyncio.create_task(sess.post(p.http_url + path, json=pre))
                async with sess.post(d + path, json=dec) as r_dec:
                    async for chunk in r_dec.content.iter_any():
                        yield chunk
                (await t_pre).release()
        finally:
            p.inflight -= 1
            self.decode_inflight[d] -= 1


def build_router_app(args: RouterArgs):
    lb = MiniLoadBalancer(args)
    app = FastAPI(title="sglang PD router")
    app.state.lb = lb

    async def route(request: Request, path: str):
        body = await request.json()
        try:
            if body.get("stream"):
                return StreamingResponse(lb.forward_stream(path, body), media_type="text/event-stream")
            status, out = await lb.forward(path, body)
            return JSONResponse(out, status_code=status)
        except RuntimeError as e:
            return JSONResponse({"error": {"message": str(e)}}, status_code=503)

    @app.get("/health")
    async def health():
        lb.refresh_prefills()
        ok = bool(lb.prefills) and bool(lb.decode_urls)
        return JSONResponse({"prefill": [p.http_url for p in lb.prefills], "decode": lb.decode_urls,
                             "routed": lb.routed}, status_code=200 if ok else 503)

    @app.post("/generate")
    async def generate(request: Request):
        return await route(request, "/generate")

    @app.post("/v1/completions")
    async def completions(request: Request):
        return await route(request, "/v1/completions")

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        return await route(request, "/v1/chat/completions")

    @app.get("/v1/models")
    async def models():
        async with aiohttp.ClientSession() as sess:
            async with sess.get(lb.decode_urls[0] + "/v1/models") as r:
                return JSONResponse(await r.json(content_type=None), status_code=r.status)

    @app.get("/get_server_info")
    async def info():
        out = {}
        async with aiohttp.ClientSession() as sess:
            for name, urls in (("prefill", [p.http_url for p in lb.prefills]), ("decode", lb.decode_urls)):
                out[name] = []
                for u in urls:
                    try:
                        async with sess.get(u + "/get_server_info") as r:
                            out[name].append(await r.json(content_type=None))
                    except Exception as e:  # noqa: BLE001
                        out[name].append({"url": u, "error": str(e)})
        return out

    return app
