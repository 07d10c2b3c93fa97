"""Model worker: owns a `ModelRunner` and turns a `ModelWorkerBatch` into sampled tokens.

Reference: `python/sgl_jax/srt/managers/tp_worker.py:61-822` (`ModelWorker`, limits derived
at :150-164 / :244, `forward_batch_generation` :468, `MockModelWorker` :722).  The reference
is single-controller: one process feeds every device of the mesh.  Here there is one worker
process per GPU; the worker on tensor-rank 0 lives beside the scheduler and broadcasts each
step's batch to the follower ranks, which run `run_tp_follower` below.
"""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Any

import threading

import numpy as np
import torch

from ..configs.model_config import ModelConfig
from ..managers.schedule_batch import ForwardMode, ModelWorkerBatch
from ..model_executor.model_runner import ModelRunner
from ..parallel import state as ps

logger = logging.getLogger(__name__)


@dataclass
class GenerationBatchResult:
    logits_output: Any
    next_token_ids: Any              # device tensor (or numpy once resolved)
    bid: int = 0
    cache_miss_count: int = 0
    extend_input_len_per_req: list | None = None
    extend_logprob_start_len_per_req: list | None = None
    accept_lens: Any = None
    copy_done: Any = None            # CUDA event: D2H of `next_token_ids_cpu` finished
    next_token_ids_cpu: Any = None
    forward_batch: Any = None
    routed_experts: Any = None       # (pinned host tensor [layers, tokens, top_k], event) of the capturer


class _Control:
    """Non-batch messages rank 0 sends to follower ranks."""

    def __init__(self, kind: str, payload: Any = None):
        self.kind = kind
        self.payload = payload


class ModelWorker:
    def __init__(self, server_args, model_config: ModelConfig | None = None, is_draft_worker: bool = False,
                 req_to_token_pool=None, token_to_kv_pool=None, max_total_num_tokens=None, model_path=None):
        self.server_args = server_args
        st = ps.get_state()
        self.tp_rank = st.tp.rank
        self.tp_size = st.tp.size
        self.model_config = model_config or ModelConfig.from_server_args(
            server_args, model_path=model_path or server_args.model_path, is_draft_model=is_draft_worker)
        self.model_runner = ModelRunner(self.model_config, server_args, st.device,
                                        req_to_token_pool=req_to_token_pool, is_draft_worker=is_draft_worker,
                                        token_to_kv_pool=token_to_kv_pool, max_total_num_tokens=max_total_num_tokens)
        self.device = self.model_runner.device
        self.max_total_num_tokens = self.model_runner.max_total_num_tokens
        self.max_prefill_tokens = server_args.max_prefill_tokens
        self.max_running_requests = self.model_runner.max_running_requests
        # longest request (prompt + output) one row can hold
        self.max_req_len = min(self.model_config.context_len - 1, self.max_total_num_tokens - 1)
        self.max_req_input_len = self.max_req_len - 5
        self.random_seed = server_args.random_seed
        self.broadcast_batches = self.tp_size > 1 and self.tp_rank == 0 and not is_draft_worker
        # rank 0 -> followers: shared-memory ring on one node, host broadcast across nodes (created by every
        # rank at the same point of its start-up; the speculative draft worker shares the target's)
        self.channel = getattr(st, "step_channel", None)
        if self.tp_size > 1 and not is_draft_worker:
            from ..parallel.step_channel import StepChannel
            mode = os.environ.get("SGLB_STEP_CHANNEL", "shm")
            multi_node = getattr(server_args, "nnodes", 1) > 1
            # several nodes (or SGLB_STEP_CHANNEL=zmq): rank 0 publishes the steps at the address the ranks
            # rendezvous on; one node: shared-memory ring
            host = None
            if multi_node or mode == "zmq":
                host = (server_args.dist_init_addr or "127.0.0.1").rsplit(":", 1)[0]
            self.channel = StepChannel(st.tp, use_shm=not multi_node and mode == "shm",
                                       timeout_s=float(server_args.dist_timeout or 120.0), pubsub_host=host)
            st.step_channel = self.channel
        self._pinned_ids = None
        self.marks: dict = {}
        # Host collectives with the follower ranks are issued from the scheduler thread (batches)
        # and from API threads (marks, reports, adapter loads): one transaction at a time, or two
        # threads would interleave collectives on the same process group in different orders.
        self._comm_lock = threading.RLock()

    # ------------------------------------------------------------------
    def get_worker_info(self):
        return (self.max_total_num_tokens, self.max_prefill_tokens, self.max_running_requests,
                self.max_req_len, self.max_req_input_len, self.random_seed, str(self.device),
                self.model_runner.req_to_token_pool.size, self.model_runner.req_to_token_pool.max_context_len)

    def get_memory_pool(self):
        return self.model_runner.req_to_token_pool, self.model_runner.token_to_kv_pool

    def get_pad_input_ids_func(self):
        return getattr(self.model_runner.model, "pad_input_ids", None)

    @property
    def sliding_window_size(self):
        return self.model_config.sliding_window

    # ------------------------------------------------------------------
    def spec_broadcast(self, kind: str, payload) -> None:
        """Ship one speculative step's host inputs to the follower ranks, which run the same
        draft / verify sequence on their shards."""
        if self.broadcast_batches:
            with self._comm_lock:
                self.channel.send(_Control(kind, payload))

    def forward_batch_generation(self, batch: ModelWorkerBatch, launch_done=None, skip_sample: bool = False,
                                 broadcast: bool = True) -> GenerationBatchResult:
        if self.broadcast_batches and broadcast and self.device.type == "cpu":
            # on CPU the model's collectives and the host-side ones (marks, reports) share one gloo group: a whole
            # step is one transaction, or another thread's collective could land between this step's
            with self._comm_lock:
                self.channel.send(batch)
                out, ids, fb = self.model_runner.forward(batch, skip_sample=skip_sample)
        else:
            if self.broadcast_batches and broadcast:
                with self._comm_lock:
                    self.channel.send(batch)
            out, ids, fb = self.model_runner.forward(batch, skip_sample=skip_sample)
        res = GenerationBatchResult(out, ids, bid=batch.bid, forward_batch=fb)
        cap = getattr(self.model_runner, "routed_capturer", None)
        if cap is not None and getattr(batch, "return_routed_experts", False):
            res.routed_experts = cap.snapshot(len(batch.input_ids))
        if ids is not None and self.device.type == "cuda":
            # start the D2H copy right away; the scheduler waits on the event when it needs the ids
            n = ids.numel()
            buf = torch.empty(n, dtype=torch.int32, pin_memory=True)
            buf.copy_(ids, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            res.next_token_ids_cpu, res.copy_done = buf, ev
        if launch_done is not None:
            launch_done.set()
        return res

    def resolve(self, res: GenerationBatchResult) -> np.ndarray:
        """Host copy of the sampled ids (blocks until the step has finished)."""
        if res.next_token_ids is None:
            return np.empty(0, np.int32)
        if res.copy_done is not None:
            res.copy_done.synchronize()
            return res.next_token_ids_cpu.numpy()
        return res.next_token_ids.cpu().numpy().astype(np.int32)

    def forward_batch_embedding(self, batch: ModelWorkerBatch):
        if self.broadcast_batches:
            with self._comm_lock:
                self.channel.send(_Control("embed", batch))
        batch.capture_hidden_mode = 1
        out, _, _ = self.model_runner.forward(batch, skip_sample=True)
        return out.hidden_states

    def load_lora_adapter(self, recv) -> tuple[bool, str]:
        from ..lora.lora_registry import LoRARef
        lm = self.model_runner.lora_manager
        if lm is None:
            return False, "LoRA is not enabled (--enable-lora)"
        if self.broadcast_batches:
            with self._comm_lock:
                self.channel.send(_Control("load_lora", recv))
        return lm.load_adapter(LoRARef(lora_id=recv.lora_id, lora_name=recv.lora_name, lora_path=recv.lora_path))

    def unload_lora_adapter(self, recv) -> tuple[bool, str]:
        lm = self.model_runner.lora_manager
        if lm is None:
            return False, "LoRA is not enabled (--enable-lora)"
        if self.broadcast_batches:
            with self._comm_lock:
                self.channel.send(_Control("unload_lora", recv))
        return lm.unload_adapter(recv.lora_id)

    def send_control(self, kind: str, payload=None):
        if self.broadcast_batches:
            with self._comm_lock:
                self.channel.send(_Control(kind, payload))

    def flush(self):
        self.send_control("flush")

    def shutdown(self):
        self.send_control("shutdown")
        if self.broadcast_batches and self.channel is not None:
            self.channel.close()

    def mark(self, tag: str):
        """Record a timing event on this rank's stream and on every follower's."""
        with self._comm_lock:
            self.send_control("mark", tag)
            _sync_all(self.device)
            self.marks[tag] = _record_event(self.device)

    def elapsed_ms_max_over_ranks(self, start_tag: str, end_tag: str) -> float:
        with self._comm_lock:
            self.send_control("report", (start_tag, end_tag))
            return report_elapsed_max(self, start_tag, end_tag)


def _sync_all(device):
    """Device synchronize + barrier over the tensor ranks: brackets a timed region."""
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    ps.barrier(ps.get_state().tp)


def _record_event(device):
    if device.type != "cuda":
        import time
        return time.perf_counter()
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    return ev


def report_elapsed_max(worker: "ModelWorker", start_tag: str, end_tag: str) -> float:
    """Device time between two marks in ms, max over the tensor ranks (every rank calls this)."""
    a, b = worker.marks[start_tag], worker.marks[end_tag]
    if worker.device.type == "cuda":
        b.synchronize()
        ms = a.elapsed_time(b)
    else:
        ms = (b - a) * 1e3
    tp = ps.get_state().tp
    if tp.size > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=tp.cpu_group)
        ms = float(t.item())
    return ms


def run_tp_follower(server_args, worker: ModelWorker | None = None, on_message=None):
    """Event loop of tensor ranks > 0: execute whatever rank 0 broadcasts."""
    worker = worker or ModelWorker(server_args)
    tp = ps.get_state().tp
    spec = None
    if server_args.speculative_algorithm is not None:
        from ..speculative.spec_info import create_spec_worker
        spec = create_spec_worker(server_args, worker)
    while True:
        try:
            msg = worker.channel.recv(on_idle=on_message)
        except EOFError:
            break
        if on_message is not None:
            on_message()          # liveness hook (e.g. re-arm a hang watchdog)
        if isinstance(msg, _Control):
            if msg.kind == "shutdown":
                break
            if msg.kind == "flush":
                worker.model_runner.req_to_token_pool.page_table.zero_()
            elif msg.kind == "embed":
                msg.payload.capture_hidden_mode = 1
                worker.model_runner.forward(msg.payload, skip_sample=True)
            elif msg.kind == "mark":
                _sync_all(worker.device)
                worker.marks[msg.payload] = _record_event(worker.device)
            elif msg.kind == "report":
                report_elapsed_max(worker, *msg.payload)
            elif msg.kind == "spec_prefill":
                spec.prefill_core(*msg.payload)
            elif msg.kind == "spec_decode":
                spec.decode_core(*msg.payload)
            elif msg.kind == "load_lora":
                from ..lora.lora_registry import LoRARef
                r = msg.payload
                worker.model_runner.lora_manager.load_adapter(
                    LoRARef(lora_id=r.lora_id, lora_name=r.lora_name, lora_path=r.lora_path))
            elif msg.kind == "unload_lora":
                worker.model_runner.lora_manager.unload_adapter(msg.payload.lora_id)
            elif msg.kind.startswith("pd_"):
                # KV hand-over of this rank's shard between a prefill and a decode engine
                from ..disaggregation.tp_mirror import handle_follower_control
                handle_follower_control(worker, msg.kind, msg.payload)
            continue
        worker.model_runner.forward(msg)
    return worker


class MockModelWorker:
    """Scheduler-test stand-in: no model, deterministic fake tokens
    (reference `tp_worker.py:722`)."""

    def __init__(self, server_args=None, max_total_num_tokens=4096, max_running_requests=64,
                 context_len=2048, vocab_size=1024, page_size=1, eos_after: int | None = None):
        self.server_args = server_args
        self.max_total_num_tokens = max_total_num_tokens
        self.max_prefill_tokens = 16384
        self.max_running_requests = max_running_requests
        self.max_req_len = context_len - 1
        self.max_req_input_len = context_len - 6
        self.random_seed = 42
        self.device = torch.device("cpu")
        self.vocab_size = vocab_size
        self.page_size = page_size
        self.tp_size = 1
        self.tp_rank = 0
        from ..mem_cache.memory_pool import ReqToTokenPool
        self.req_to_token_pool = ReqToTokenPool(max_running_requests + 8, context_len + 8, "cpu", page_size)
        self.model_config = type("MC", (), {"vocab_size": vocab_size, "context_len": context_len,
                                            "hf_eos_token_id": set(), "is_embedding": False,
                                            "sliding_window": None, "num_experts": None})()
        self.forward_ct = 0
        self.batches: list[ModelWorkerBatch] = []
        self.future_map = np.zeros(self.req_to_token_pool.size + 2, np.int32)

    def get_worker_info(self):
        return (self.max_total_num_tokens, self.max_prefill_tokens, self.max_running_requests, self.max_req_len,
                self.max_req_input_len, self.random_seed, "cpu", self.req_to_token_pool.size,
                self.req_to_token_pool.max_context_len)

    def get_memory_pool(self):
        return self.req_to_token_pool, None

    def forward_batch_generation(self, batch: ModelWorkerBatch, launch_done=None, skip_sample=False):
        self.forward_ct += 1
        self.batches.append(batch)
        # next token = (sum of the sequence's current length and last input id) mod vocab: cheap,
        # deterministic and independent of batch composition
        input_ids = np.asarray(batch.input_ids).copy()
        neg = input_ids < 0
        if neg.any():   # overlap mode: placeholders -slot resolve through the future map
            input_ids[neg] = self.future_map[-input_ids[neg]]
        if batch.forward_mode.is_extend():
            last = np.cumsum(batch.extend_seq_lens) - 1
            last_ids = input_ids[last]
        else:
            last_ids = input_ids
        ids = ((last_ids.astype(np.int64) * 31 + batch.seq_lens) % self.vocab_size).astype(np.int32)
        if batch.future_slots is not None:
            self.future_map[np.asarray(batch.future_slots)] = ids
        if launch_done is not None:
            launch_done.set()
        return GenerationBatchResult(None, ids, bid=batch.bid)

    def resolve(self, res):
        return np.asarray(res.next_token_ids)

    def send_control(self, *a, **k):
        pass

    def flush(self):
        pass

    def shutdown(self):
        pass
