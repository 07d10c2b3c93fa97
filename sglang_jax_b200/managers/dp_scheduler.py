"""Data-parallel attention under ONE scheduler.

Reference: one `Scheduler` drives a `("data", "tensor")` mesh; every batch is laid out as `dp_size` equal
sections, each with its own KV allocator and radix-tree namespace, and requests are routed to a section by
one of four policies (`python/sgl_jax/srt/managers/schedule_batch.py:722` `ScheduleReqsInfo`, `:2038`
`_compute_global_padding_sizes`, `managers/scheduler.py:722-1062`, `mem_cache/allocator.py:161`,
`mem_cache/radix_cache.py:31`).  `tp_size` is the total device count, a section runs on `tp_size / dp_size`
of them.

Here there is one process per GPU.  The world is laid out `[dp, tensor]` row-major; the scheduler process is
the leader of section 0, the first rank of every other section is that section's leader (`run_dp_leader`)
and the remaining ranks are ordinary tensor-parallel followers of their leader.  The one scheduler keeps, per
section, the waiting queue, the running batch, the request -> slot table, the page allocator and the prefix
tree (`SectionScheduler`: the same logic a single-section engine runs), routes every arriving request to a
section (`dp_schedule_policy`), and advances all sections in lock-step: in each iteration every section forms
its next batch and launches it, on this process's GPU for section 0 and through a shared-memory ring to the
section's leader otherwise; sampled tokens (and log-probabilities when asked for) come back through one ring
per leader.  With overlap scheduling a section's results are read one iteration later, so the sections'
forwards of one iteration run concurrently on their GPUs.  Sections pad nothing to a common shape: each
replays its own captured graph bucket.

Expert parallelism, when enabled together with `dp_size > 1`, spans the ranks of one section.
"""

from __future__ import annotations

import dataclasses
import logging
import os
import pickle
import queue
import threading
import time
import uuid
from types import SimpleNamespace

import numpy as np

from .dp_schedule_policy import DPRankAssignment, DPRankLoad, create_dp_schedule_policy
from .io_struct import (AbortReq, FlushCacheReqInput, FlushCacheReqOutput, TokenizedEmbeddingReqInput,
                        TokenizedGenerateReqInput)
from .scheduler import Scheduler

logger = logging.getLogger(__name__)

RESULT_SLOT_BYTES = 1 << 20
RESULT_SLOTS = 8
KIND_IDS = 1
KIND_OBJ = 0
KIND_PART = 2


class _SectionCaches:
    """The sections' prefix trees behind the one-tree interface the cache-aware policy expects: the `dp_rank`
    of the key selects the tree."""

    def __init__(self, caches):
        self.caches = caches
        self.disable = any(getattr(c, "disable", True) for c in caches)

    def match_prefix(self, key):
        return self.caches[key.dp_rank or 0].match_prefix(key)


class SectionScheduler(Scheduler):
    """One data-parallel section: a `Scheduler` fed by the router of `DPScheduler` instead of a socket."""

    def __init__(self, server_args, dp_rank: int, tp_worker, owner: "DPScheduler", tokenizer=None, model_config=None):
        self.section_rank = dp_rank
        self.owner = owner
        self.inbox: queue.Queue = queue.Queue()
        # prompt tokens routed here that the section has not taken out of its inbox yet: a burst that arrives in one
        # intake tick is balanced against what the same tick already sent (reference `dp_rank_assignment.py`)
        self.inbox_tokens = 0
        super().__init__(server_args, None, tp_worker=tp_worker, recv_queue=self.inbox, send_queue=None,
                         tokenizer=tokenizer, model_config=model_config)

    def send_to_detokenizer(self, obj):
        self.owner.front.send_to_detokenizer(obj)

    def send_to_tokenizer(self, obj):
        self.owner.front.send_to_tokenizer(obj)

    def handle_generate_request(self, recv):
        recv.dp_rank = self.section_rank
        self.inbox_tokens = max(self.inbox_tokens - len(recv.input_ids or ()), 0)
        return super().handle_generate_request(recv)

    def on_idle(self):
        # the owner sleeps once when every section is idle
        self.check_memory()
        self.new_token_ratio = self.init_new_token_ratio

    def get_load(self) -> dict:
        d = super().get_load()
        d["dp_rank"] = self.section_rank
        return d

    def load(self) -> DPRankLoad:
        used, _ = self.token_usage()
        return DPRankLoad(running=len(self.running_batch.reqs), queued=len(self.waiting_queue) + self.inbox.qsize(),
                          queued_tokens=sum(len(r.origin_input_ids) for r in self.waiting_queue) + self.inbox_tokens,
                          used_tokens=used)


class _FrontDoor(Scheduler):
    """Only the IPC endpoints of a `Scheduler` (sockets or queues): what the sections share."""

    def __init__(self, server_args, port_args, recv_queue, send_queue):    # the rest of Scheduler is not built
        self.server_args, self.port_args = server_args, port_args
        self._init_ipc(recv_queue, send_queue)


class DPScheduler:
    """`dp_size` sections advanced in lock-step by one loop."""

    def __init__(self, server_args, port_args=None, workers=None, recv_queue=None, send_queue=None, tokenizer=None,
                 model_config=None):
        self.server_args = server_args
        self.dp_size = server_args.dp_size
        assert workers is not None and len(workers) == self.dp_size, "one worker handle per section"
        self.front = _FrontDoor(server_args, port_args, recv_queue, send_queue)
        self.sections = [SectionScheduler(server_args, d, workers[d], self, tokenizer=tokenizer,
                                          model_config=model_config) for d in range(self.dp_size)]
        s0 = self.sections[0]
        self.policy = create_dp_schedule_policy(server_args.dp_schedule_policy or "round_robin", self.dp_size)
        self.assignment = DPRankAssignment(self.dp_size)
        self.routed = [0] * self.dp_size
        self.caches = _SectionCaches([s.tree_cache for s in self.sections])
        # what the engine's front door reads
        self.tokenizer = s0.tokenizer
        self.model_config = s0.model_config
        self.max_total_num_tokens = sum(s.max_total_num_tokens for s in self.sections)
        self.max_req_input_len = min(s.max_req_input_len for s in self.sections)
        self.enable_overlap = all(s.enable_overlap for s in self.sections)
        for s in self.sections:
            s.enable_overlap = self.enable_overlap
        self.tp_worker = s0.tp_worker
        self.step_hooks: list = []
        self.iterations = 0

    # ------------------------------------------------------------------ routing
    def select_dp_for_request(self, recv) -> int:
        """Reference `scheduler.py:1043`: an explicit `dp_rank` wins, a request id that already has a section
        keeps it, otherwise the policy decides from the sections' loads and prefix trees."""
        pinned = getattr(recv, "dp_rank", None)
        if pinned is not None and 0 <= int(pinned) < self.dp_size:
            return int(pinned)
        known = self.assignment.get(recv.rid)
        if known is not None:
            return known
        ids = list(recv.input_ids or [])
        stub = SimpleNamespace(origin_input_ids=ids, extend_input_len=len(ids), extra_key=getattr(recv, "extra_key", None))
        return self.policy.select(stub, [s.load() for s in self.sections], self.caches)

    def dispatch(self, msgs: list):
        for m in msgs:
            if isinstance(m, (TokenizedGenerateReqInput, TokenizedEmbeddingReqInput)):
                d = self.select_dp_for_request(m)
                self.assignment.assign(m.rid, d)
                self.routed[d] += 1
                if isinstance(m, TokenizedGenerateReqInput):
                    self.sections[d].inbox_tokens += len(m.input_ids or ())
                self.sections[d].inbox.put(m)
            elif isinstance(m, AbortReq):
                for s in self.sections:
                    s.inbox.put(m)
            elif isinstance(m, FlushCacheReqInput):
                res = [s.flush_cache() for s in self.sections]
                ok = all(r[0] for r in res)
                self.front.send_to_tokenizer(FlushCacheReqOutput(
                    success=ok, flushed_items=sum(r[1] for r in res),
                    error_msg="" if ok else "Cache not flushed because there are pending requests."))
            else:
                # control messages apply to every section; section 0 answers
                for s in self.sections[1:]:
                    fn = s._dispatch.get(type(m))
                    if fn is not None:
                        fn(m)
                self.sections[0].inbox.put(m)

    # ------------------------------------------------------------------ loop
    def step(self) -> bool:
        self.dispatch(self.front.recv_requests())
        ran = False
        for s in self.sections:
            ran |= bool(s.step_overlap() if self.enable_overlap else s.step_normal())
        self.iterations += 1
        if (self.iterations & 1023) == 0:
            live = {r.rid for s in self.sections for r in list(s.running_batch.reqs) + s.waiting_queue}
            for rid in [r for r in self.assignment.table if r not in live]:
                self.assignment.release(rid)
        if not ran and all(not s.result_queue for s in self.sections):
            time.sleep(0.0005)
        for h in self.step_hooks:
            h(self, None)
        return ran

    def event_loop(self, stop_event: threading.Event | None = None):
        while not (stop_event is not None and stop_event.is_set()):
            self.step()

    event_loop_overlap = event_loop
    event_loop_normal = event_loop

    def shutdown(self):
        for s in self.sections:
            s.shutdown()
        ch = getattr(self.sections[0].tp_worker, "dp_channel", None)
        if ch is not None:
            ch.close()

    def get_load(self) -> list[dict]:
        return [s.get_load() for s in self.sections]

    # introspection shared with `Scheduler`
    @property
    def running_batch(self):
        return self.sections[0].running_batch

    @property
    def waiting_queue(self):
        return [r for s in self.sections for r in s.waiting_queue]

    @property
    def tree_cache(self):
        return self.sections[0].tree_cache

    @property
    def forward_ct(self):
        return sum(s.forward_ct for s in self.sections)


# ------------------------------------------------------------------------------------------ remote sections
def _push_obj(ring, obj, timeout_s: float) -> bool:
    blob = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
    n = ring.slot_bytes()
    while len(blob) > n:
        head, blob = blob[:n], blob[n:]
        if not ring.push(head, KIND_PART, timeout_s):
            return False
    return ring.push(blob, KIND_OBJ, timeout_s)


def _pop_msg(ring, poll_s: float):
    """`None` on time-out, else `(kind, payload)` with pickled messages re-assembled and loaded."""
    parts = []
    while True:
        got = ring.pop(poll_s, True)
        if got is None:
            if parts and not ring.closed():
                continue
            return None
        kind, payload = got
        if kind == KIND_IDS:
            return kind, np.asarray(payload, np.int32)
        if kind == KIND_PART:
            parts.append(payload)
            continue
        return kind, pickle.loads(b"".join(parts) + payload if parts else payload)


def _host_logits(lo):
    """The log-probability fields of a `LogitsProcessorOutput` as host tensors (full logits stay on the device)."""
    import torch
    if lo is None:
        return None
    kw = {}
    for f in dataclasses.fields(lo):
        v = getattr(lo, f.name)
        if f.name == "next_token_logits":
            v = None
        elif isinstance(v, torch.Tensor):
            v = v.detach().cpu()
        kw[f.name] = v
    return type(lo)(**kw)


class RemoteSectionWorker:
    """The scheduler's handle on a section whose leader is another process: batches go out through the
    channel to the leaders (tagged with the section), results come back through the leader's ring.  The host
    side of the section's request -> slot table lives here, with the scheduler."""

    def __init__(self, dp_rank: int, channel, in_ring, info: dict, model_config, page_size: int, lock):
        from ..mem_cache.memory_pool import ReqToTokenPool
        self.dp_rank = dp_rank
        self.channel, self.in_ring = channel, in_ring
        self.info = info
        self.model_config = model_config
        self.device = "cpu"
        self.req_to_token_pool = ReqToTokenPool(info["pool_rows"], info["pool_width"], "cpu", page_size)
        self.pending: dict[int, tuple] = {}
        self._lock = lock
        self.timeout_s = 300.0

    def get_worker_info(self):
        i = self.info
        return (i["max_total_num_tokens"], i["max_prefill_tokens"], i["max_running_requests"], i["max_req_len"],
                i["max_req_input_len"], i["random_seed"], "cpu", i["pool_rows"], i["pool_width"])

    def get_memory_pool(self):
        return self.req_to_token_pool, None

    def get_pad_input_ids_func(self):
        return None

    def forward_batch_generation(self, batch, launch_done=None, skip_sample=False):
        from .tp_worker import GenerationBatchResult
        batch.dp_rank = self.dp_rank
        with self._lock:
            self.channel.send(batch)
        if launch_done is not None:
            launch_done.set()
        return GenerationBatchResult(None, batch.bid, bid=batch.bid)

    def forward_batch_embedding(self, batch):
        from .tp_worker import _Control
        batch.dp_rank = self.dp_rank
        with self._lock:
            self.channel.send(_Control("embed", batch))
        return self._wait(batch.bid)[1]

    def _wait(self, bid: int):
        t0 = time.time()
        while bid not in self.pending:
            got = _pop_msg(self.in_ring, 1.0)
            if got is None:
                if self.in_ring.closed() or time.time() - t0 > self.timeout_s:
                    raise RuntimeError(f"no result from the leader of data-parallel section {self.dp_rank}")
                continue
            kind, payload = got
            if kind == KIND_IDS:
                self.pending[int(payload[0])] = (payload[1:], None)
            else:
                self.pending[int(payload["bid"])] = (payload["ids"], payload.get("out"))
        return self.pending.pop(bid)

    def resolve(self, res) -> np.ndarray:
        if res.next_token_ids_cpu is not None:
            return res.next_token_ids_cpu
        ids, out = self._wait(res.bid)
        res.next_token_ids_cpu = np.asarray(ids, np.int32)
        if out is not None:
            res.logits_output = out
        return res.next_token_ids_cpu

    def send_control(self, kind, payload=None):
        from .tp_worker import _Control
        with self._lock:
            self.channel.send(_Control(kind, {"dp_rank": self.dp_rank, "payload": payload}))

    def flush(self):
        self.send_control("flush")

    def shutdown(self):
        try:
            self.send_control("shutdown")
        except Exception:
            pass


def _needs_rich_result(batch) -> bool:
    return bool(getattr(batch, "return_logprob", False) or getattr(batch, "capture_hidden_mode", 0)
                or getattr(batch, "return_routed_experts", False))


def connect_sections(server_args, local_worker) -> list:
    """On the scheduler's rank: the worker handle of every section (`local_worker` for section 0).  The
    counterpart of the hand-shake at the top of `run_dp_leader`; both run right after `ModelWorker` is built."""
    from ..mem_cache import _sched_native as sn
    from ..parallel import state as ps
    from ..parallel.step_channel import StepChannel
    st = ps.get_state()
    dp = st.dp
    assert dp.rank == 0 and dp.size == server_args.dp_size
    channel = StepChannel(dp, use_shm=True, timeout_s=float(server_args.dist_timeout or 120.0))
    if channel.ring is None:
        raise RuntimeError("data-parallel attention needs the shared-memory step ring (one node)")
    tag = ps.broadcast_object(f"{os.getpid()}_{uuid.uuid4().hex[:8]}", src=0, group=dp)
    ps.barrier(dp)                      # the leaders have created their result rings
    lock = threading.Lock()
    workers = [local_worker]
    for d in range(1, dp.size):
        ring = sn.StepRing(f"/sglb_dpres_{tag}_{d}", RESULT_SLOTS, RESULT_SLOT_BYTES, 1, 0)
        got = None
        t0 = time.time()
        while got is None:
            got = _pop_msg(ring, 1.0)
            if got is None and time.time() - t0 > 600:
                raise RuntimeError(f"the leader of data-parallel section {d} did not report its pool limits")
        workers.append(RemoteSectionWorker(d, channel, ring, got[1], local_worker.model_config,
                                           server_args.page_size, lock))
    local_worker.dp_channel = channel
    return workers


def run_dp_leader(server_args, on_message=None):
    """Event loop of the first rank of a section other than section 0: runs the section's batches (passing
    them on to its own tensor-parallel followers) and returns what was sampled."""
    from ..mem_cache import _sched_native as sn
    from ..parallel import state as ps
    from ..parallel.step_channel import StepChannel
    from .schedule_batch import ModelWorkerBatch
    from .tp_worker import ModelWorker, _Control
    st = ps.get_state()
    dp_rank = st.dp.rank
    worker = ModelWorker(server_args)
    channel = StepChannel(st.dp, use_shm=True, timeout_s=float(server_args.dist_timeout or 120.0))
    tag = ps.broadcast_object(None, src=0, group=st.dp)
    out_ring = sn.StepRing(f"/sglb_dpres_{tag}_{dp_rank}", RESULT_SLOTS, RESULT_SLOT_BYTES, 1)
    ps.barrier(st.dp)
    if channel.ring is None:
        raise RuntimeError("data-parallel attention needs the shared-memory step ring (one node)")
    mr = worker.model_runner
    _push_obj(out_ring, dict(max_total_num_tokens=worker.max_total_num_tokens,
                             max_prefill_tokens=worker.max_prefill_tokens,
                             max_running_requests=worker.max_running_requests, max_req_len=worker.max_req_len,
                             max_req_input_len=worker.max_req_input_len, random_seed=worker.random_seed,
                             pool_rows=mr.req_to_token_pool.size, pool_width=mr.req_to_token_pool.max_context_len), 60.0)
    def finish(item) -> bool:
        b, res = item
        ids = np.asarray(worker.resolve(res), np.int32)
        if _needs_rich_result(b):
            return _push_obj(out_ring, {"bid": b.bid, "ids": ids, "out": _host_logits(res.logits_output)}, 60.0)
        return out_ring.push_ints(np.concatenate([np.asarray([b.bid], np.int32), ids]), KIND_IDS, 60.0)

    inflight = None          # (batch, result) launched but not yet reported
    while True:
        try:
            # with a step in flight, look for the next one first: the scheduler sends step n+1 before it reads
            # step n (overlap scheduling), and launching it now keeps this GPU's queue non-empty
            msg = channel.recv(poll_s=0.0, block=False) if inflight is not None else channel.recv(on_idle=on_message)
        except EOFError:
            break
        if msg is None:
            ok, inflight = finish(inflight), None
            if not ok:
                logger.error("the scheduler stopped reading results of section %d", dp_rank)
                break
            continue
        if on_message is not None:
            on_message()
        if isinstance(msg, _Control):
            p = msg.payload
            target = p.get("dp_rank") if isinstance(p, dict) else getattr(p, "dp_rank", None)
            if target is not None and target != dp_rank:
                continue
            if inflight is not None:
                finish(inflight)
                inflight = None
            if msg.kind == "shutdown":
                break
            if msg.kind == "flush":
                mr.req_to_token_pool.page_table.zero_()
                worker.flush()
            elif msg.kind == "embed":
                emb = worker.forward_batch_embedding(p)
                _push_obj(out_ring, {"bid": p.bid, "ids": None, "out": emb.cpu() if hasattr(emb, "cpu") else emb}, 60.0)
            continue
        if not isinstance(msg, ModelWorkerBatch) or msg.dp_rank != dp_rank:
            continue
        res = worker.forward_batch_generation(msg)
        prev, inflight = inflight, (msg, res)
        if prev is not None and not finish(prev):
            break
    out_ring.close()
    worker.shutdown()
    return worker
