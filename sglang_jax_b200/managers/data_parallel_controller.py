"""Data parallelism: `dp_size` engine replicas (each a tensor-parallel group of
`tp_size / dp_size` GPUs with its own scheduler, KV pool and prefix cache) behind one front door
that routes every request with the configured policy.

The reference keeps one scheduler and lays each batch out as `dp_size` sections of one SPMD
program (`python/sgl_jax/srt/managers/schedule_batch.py:722-835`, routing in
`scheduler.py:722-1062`).  With one process per GPU there is no shared program to lay sections
into; replicas that schedule independently give the same capacity and the same four routing
policies, and a slow prefill in one replica does not stall the decode steps of another."""

from __future__ import annotations

import copy
import threading
from concurrent.futures import ThreadPoolExecutor
from types import SimpleNamespace

from .dp_schedule_policy import DPRankAssignment, DPRankLoad, create_dp_schedule_policy


class DataParallelEngine:
    def __init__(self, server_args):
        from ..entrypoints.engine import Engine
        dp = server_args.dp_size
        per = server_args.tp_size // dp
        self.server_args = server_args
        self.replicas = []
        base = list(server_args.device_indexes) if server_args.device_indexes else list(range(server_args.tp_size))
        for r in range(dp):
            sa = copy.copy(server_args)
            sa.dp_size, sa.tp_size = 1, per
            sa.ep_size = min(server_args.ep_size, per)
            sa.device_indexes = base[r * per:(r + 1) * per]
            sa.port = server_args.port + 100 * (r + 1)
            self.replicas.append(Engine(server_args=sa, _replica=True))
        self.policy = create_dp_schedule_policy(server_args.dp_schedule_policy, dp)
        self.loads = [DPRankLoad() for _ in range(dp)]
        self.assignment = DPRankAssignment(dp)
        self.routed = [0] * dp
        self._lock = threading.Lock()
        self._pool = ThreadPoolExecutor(max_workers=dp)
        self.tokenizer_manager = self.replicas[0].tokenizer_manager

    # ------------------------------------------------------------------ routing
    def _route(self, n_tokens: int, ids) -> int:
        stub = SimpleNamespace(origin_input_ids=list(ids) if ids is not None else [0] * n_tokens,
                               extend_input_len=n_tokens, extra_key=None)
        caches = [getattr(getattr(e, "scheduler", None), "tree_cache", None) for e in self.replicas]
        with self._lock:
            try:
                r = self.policy.select(stub, self.loads, caches if all(c is not None for c in caches) else None)
            except TypeError:
                r = self.policy.select(stub, self.loads)
            self.loads[r].queued += 1
            self.loads[r].queued_tokens += n_tokens
            self.routed[r] += 1
        return r

    def _done(self, r: int, n_tokens: int):
        with self._lock:
            self.loads[r].queued = max(0, self.loads[r].queued - 1)
            self.loads[r].queued_tokens = max(0, self.loads[r].queued_tokens - n_tokens)

    # ------------------------------------------------------------------ generation
    def generate(self, prompt=None, sampling_params=None, input_ids=None, **kw):
        single = isinstance(prompt, str) or (input_ids is not None and input_ids and isinstance(input_ids[0], int))
        prompts = [prompt] if isinstance(prompt, str) else prompt
        ids = [input_ids] if (single and input_ids is not None) else input_ids
        n = len(prompts) if prompts is not None else len(ids)
        sps = sampling_params if isinstance(sampling_params, list) else [sampling_params] * n
        plan: dict[int, list[int]] = {}
        sizes = []
        for i in range(n):
            toks = ids[i] if ids is not None else None
            nt = len(toks) if toks is not None else max(len(prompts[i]) // 4, 1)
            sizes.append(nt)
            forced = kw.get("dp_rank")
            r = forced if isinstance(forced, int) else self._route(nt, toks)
            plan.setdefault(r, []).append(i)
        kw.pop("dp_rank", None)
        per_item = {k: v for k, v in kw.items() if isinstance(v, list) and len(v) == n}

        def run(r, idx):
            sub = dict(kw)
            for k, v in per_item.items():
                sub[k] = [v[i] for i in idx]
            try:
                return self.replicas[r].generate(
                    prompt=[prompts[i] for i in idx] if prompts is not None else None,
                    sampling_params=[sps[i] for i in idx],
                    input_ids=[ids[i] for i in idx] if ids is not None else None, **sub)
            finally:
                for i in idx:
                    self._done(r, sizes[i])

        futs = {r: self._pool.submit(run, r, idx) for r, idx in plan.items()}
        out = [None] * n
        for r, idx in plan.items():
            for i, o in zip(idx, futs[r].result()):
                o.setdefault("meta_info", {})["dp_rank"] = r
                out[i] = o
        return out[0] if single else out

    # ------------------------------------------------------------------ fan-out controls
    def flush_cache(self):
        return [e.flush_cache() for e in self.replicas]

    def get_server_info(self) -> dict:
        infos = [e.get_server_info() for e in self.replicas]
        out = dict(infos[0])
        out["internal_states"] = [s for i in infos for s in i.get("internal_states", [])]
        out["dp_routed"] = list(self.routed)
        return out

    def abort_request(self, rid: str = "", abort_all: bool = False):
        for e in self.replicas:
            e.abort_request(rid, abort_all)

    def shutdown(self):
        for e in self.replicas:
            e.shutdown()
        self._pool.shutdown(wait=False)
