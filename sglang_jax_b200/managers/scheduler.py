"""The scheduler: continuous batching with chunked prefill, prefix-cache-aware admission,
retraction under memory pressure, abort / pause / flush control and overlap scheduling.

Reference: `python/sgl_jax/srt/managers/scheduler.py:183-3037` (event loops :1064/:1113,
`get_next_batch_to_run` :1937, `get_new_batch_prefill` :2090, `update_running_batch` :2357,
`run_batch` :2456, `process_batch_result` :2584, watchdog :2724, abort :2749,
pause/continue :2859/:2909, `run_scheduler_process` :2951).

Overlap scheduling here needs no forward thread: kernel launches and CUDA-graph replays
are asynchronous, so the loop launches step n+1 (whose input ids are negative placeholders
resolved on the device from the future-token map) and only then blocks on the pinned D2H
copy of step n's tokens.
"""

from __future__ import annotations

import faulthandler
import logging
import os
import queue
import signal
import threading
import time
from collections import deque
from types import SimpleNamespace
from typing import Any

import numpy as np

from ..global_config import global_config
from ..mem_cache.allocator import PagedTokenToKVPoolAllocator, TokenToKVPoolAllocator
from ..mem_cache.chunk_cache import ChunkCache
from ..mem_cache.radix_cache import RadixCache
from ..sampling.sampling_params import SamplingParams
from .io_struct import (AbortReq, BatchTokenIDOut, CloseSessionReqInput, CloseSessionReqOutput,
                        ConfigureLoggingReq, ConfigureLoggingReqOutput, ContinueGenerationReqInput,
                        FlushCacheReqInput, FlushCacheReqOutput, GetInternalStateReq, LoadLoRAAdapterReqInput,
                        LoRAUpdateOutput, UnloadLoRAAdapterReqInput,
                        GetInternalStateReqOutput, GetLoadReqInput, GetLoadReqOutput, HealthCheckOutput,
                        OpenSessionReqInput, OpenSessionReqOutput, PauseGenerationReqInput, ProfileReq,
                        ReleaseMemoryOccupationReqInput, ReleaseMemoryOccupationReqOutput,
                        ResumeMemoryOccupationReqInput, ResumeMemoryOccupationReqOutput, SetInternalStateReq,
                        SetInternalStateReqOutput, TokenizedEmbeddingReqInput, TokenizedGenerateReqInput)
from .schedule_batch import FINISH_ABORT, ForwardMode, Req, ScheduleBatch
from .schedule_policy import AddReqResult, PrefillAdder, SchedulePolicy
from .scheduler_metrics_mixin import SchedulerMetricsMixin
from .scheduler_output_processor_mixin import SchedulerOutputProcessorMixin
from .scheduler_profiler_mixin import SchedulerProfilerMixin

logger = logging.getLogger(__name__)

# Fault injection: force a retraction every N decode steps (reference `scheduler.py:116-118`).
TEST_RETRACT = os.environ.get("SGLANG_TEST_RETRACT", "").lower() in ("1", "true")
TEST_RETRACT_INTERVAL = int(os.environ.get("SGLANG_TEST_RETRACT_INTERVAL", "3"))
TEST_RETRACT_NO_PREFILL_BS = int(os.environ.get("SGLANG_TEST_RETRACT_NO_PREFILL_BS", str(2 ** 31)))


class SyncError(RuntimeError):
    """A mirror scheduler on another node disagreed with node 0."""


from ..disaggregation.decode import SchedulerDisaggregationDecodeMixin  # noqa: E402
from ..disaggregation.prefill import SchedulerDisaggregationPrefillMixin  # noqa: E402


class SendDataError(RuntimeError):
    pass


class ReceiveDataError(RuntimeError):
    pass


class Scheduler(SchedulerOutputProcessorMixin, SchedulerMetricsMixin, SchedulerProfilerMixin,
                SchedulerDisaggregationPrefillMixin, SchedulerDisaggregationDecodeMixin):
    def __init__(self, server_args, port_args=None, tp_worker=None, recv_queue: queue.Queue | None = None,
                 send_queue: queue.Queue | None = None, tokenizer=None, model_config=None):
        self.server_args = server_args
        self.port_args = port_args
        self.page_size = server_args.page_size
        self.schedule_policy_name = server_args.schedule_policy
        self.enable_overlap = not server_args.disable_overlap_schedule
        if server_args.speculative_algorithm is not None:
            # a speculative step needs the accepted tokens of the previous one on the host
            self.enable_overlap = False
            server_args.disable_overlap_schedule = True
            server_args.enable_mixed_chunk = False
        self.stream_interval = server_args.stream_interval
        self.spec_algorithm = server_args.speculative_algorithm
        self.is_embedding = server_args.is_embedding
        self.tp_rank = 0
        self._init_ipc(recv_queue, send_queue)

        # ---- worker
        if tp_worker is None:
            from .tp_worker import ModelWorker
            tp_worker = ModelWorker(server_args, model_config)
        self.tp_worker = tp_worker
        (self.max_total_num_tokens, self.max_prefill_tokens, self.max_running_requests, self.max_req_len,
         self.max_req_input_len, self.random_seed, self.device, _, _) = tp_worker.get_worker_info()
        self.model_config = getattr(tp_worker, "model_config", model_config)
        self.vocab_size = self.model_config.vocab_size
        self.is_embedding = self.is_embedding or getattr(self.model_config, "is_embedding", False)
        self.tokenizer = tokenizer
        if self.tokenizer is None and not server_args.skip_tokenizer_init and server_args.tokenizer_path:
            try:
                from ..utils.hf_transformers_utils import get_tokenizer
                self.tokenizer = get_tokenizer(server_args.tokenizer_path, trust_remote_code=server_args.trust_remote_code)
            except Exception as e:  # the scheduler only needs it for stop strings
                logger.warning("scheduler runs without a tokenizer: %s", e)
        self.draft_worker = None
        self.spec_num_total_accepted_tokens = 0
        self.spec_num_total_forward_ct = 0
        if self.spec_algorithm is not None and hasattr(tp_worker, "model_runner"):
            from ..speculative.spec_info import create_spec_worker
            self.draft_worker = create_spec_worker(server_args, tp_worker)

        # ---- memory + cache
        self.req_to_token_pool, self.token_to_kv_pool = tp_worker.get_memory_pool()
        self.init_memory_pool_and_cache()

        # ---- queues / state
        self.waiting_queue: list[Req] = []
        self.running_batch: ScheduleBatch = self._empty_batch()
        self.cur_batch: ScheduleBatch | None = None
        self.last_batch: ScheduleBatch | None = None
        self.chunked_req: Req | None = None
        self.forward_ct = 0
        self.return_health_check_ct = 0
        self._paused = False
        self.sessions: dict[str, Any] = {}
        self.grammar_queue: list[Req] = []
        self.grammar_backend = None
        if not server_args.skip_tokenizer_init and self.tokenizer is not None:
            from ..constrained.base_grammar_backend import create_grammar_backend
            self.grammar_backend = create_grammar_backend(server_args, self.tokenizer, self.vocab_size)
        self.chunked_prefill_size = server_args.chunked_prefill_size if server_args.chunked_prefill_size > 0 else None
        self.policy = SchedulePolicy(self.schedule_policy_name, self.tree_cache)
        self.init_new_token_ratio = min(global_config.default_init_new_token_ratio *
                                        server_args.schedule_conservativeness, 1.0)
        self.min_new_token_ratio = min(self.init_new_token_ratio * global_config.default_min_new_token_ratio_factor, 1.0)
        self.new_token_ratio_decay = (self.init_new_token_ratio - self.min_new_token_ratio) / \
            global_config.default_new_token_ratio_decay_steps
        self.new_token_ratio = self.init_new_token_ratio
        self.decode_steps_since_prefill = 0
        self.decode_first_interleave = int(os.environ.get("SGL_DECODE_FIRST_INTERLEAVE", "0"))
        self.result_queue: deque = deque()
        # callables `hook(scheduler, batch_or_None)` run at the end of every loop iteration
        self.step_hooks: list = []
        self.init_metrics()
        self.init_profiler()
        self.precision_tracer_state: dict = {"enabled": False}

        # ---- watchdog
        self.watchdog_last_forward_ct = 0
        self.watchdog_last_time = time.perf_counter()
        self._watchdog_stop = threading.Event()
        self.parent_pid = os.getppid()
        if server_args.watchdog_timeout and server_args.watchdog_timeout > 0 and port_args is not None:
            threading.Thread(target=self.watchdog_thread, daemon=True).start()

        self.disagg_mode = server_args.disaggregation_mode
        if self.disagg_mode == "prefill":
            self.init_disaggregation_prefill()
        elif self.disagg_mode == "decode":
            # transferred requests enter the decode batch with a host-known first token: their first decode step is
            # fed that id instead of a placeholder (`ScheduleBatch.prepare_for_decode`), so overlap scheduling stays on
            self.init_disaggregation_decode()

        self._dispatch = {
            TokenizedGenerateReqInput: self.handle_generate_request,
            TokenizedEmbeddingReqInput: self.handle_embedding_request,
            AbortReq: self.abort_request,
            FlushCacheReqInput: self.flush_cache_wrapped,
            PauseGenerationReqInput: self.pause_generation,
            ContinueGenerationReqInput: self.continue_generation,
            GetInternalStateReq: self.get_internal_state,
            SetInternalStateReq: self.set_internal_state,
            GetLoadReqInput: lambda r: GetLoadReqOutput(**self.get_load()),
            ProfileReq: self.profile,
            LoadLoRAAdapterReqInput: self.load_lora_adapter,
            UnloadLoRAAdapterReqInput: self.unload_lora_adapter,
            OpenSessionReqInput: self.open_session,
            CloseSessionReqInput: self.close_session,
            ConfigureLoggingReq: self.configure_logging,
            ReleaseMemoryOccupationReqInput: lambda r: ReleaseMemoryOccupationReqOutput(
                r.request_id, False, "release_memory_occupation is not supported"),
            ResumeMemoryOccupationReqInput: lambda r: ResumeMemoryOccupationReqOutput(
                r.request_id, False, "resume_memory_occupation is not supported"),
        }

    # ------------------------------------------------------------------ ipc
    def _init_ipc(self, recv_queue, send_queue):
        self._recv_q = recv_queue
        self._send_q = send_queue
        self._zmq = None
        if recv_queue is None and self.port_args is not None:
            import zmq
            ctx = zmq.Context(2)
            self._zmq = ctx
            self.recv_from_tokenizer = ctx.socket(zmq.PULL)
            self.recv_from_tokenizer.bind(self.port_args.scheduler_input_ipc_name)
            self.send_to_tokenizer_sock = ctx.socket(zmq.PUSH)
            self.send_to_tokenizer_sock.connect(self.port_args.tokenizer_ipc_name)
            self.send_to_detok_sock = ctx.socket(zmq.PUSH)
            self.send_to_detok_sock.connect(self.port_args.detokenizer_ipc_name)

    def send_to_detokenizer(self, obj):
        if self._send_q is not None:
            self._send_q.put(obj)
        elif self._zmq is not None:
            self.send_to_detok_sock.send_pyobj(obj)

    def send_to_tokenizer(self, obj):
        """Control replies skip the detokenizer."""
        if self._send_q is not None:
            self._send_q.put(obj)
        elif self._zmq is not None:
            self.send_to_tokenizer_sock.send_pyobj(obj)

    def recv_requests(self) -> list:
        out = []
        if self._recv_q is not None:
            while True:
                try:
                    out.append(self._recv_q.get_nowait())
                except queue.Empty:
                    break
        elif self._zmq is not None:
            import zmq
            while True:
                try:
                    out.append(self.recv_from_tokenizer.recv_pyobj(zmq.NOBLOCK))
                except zmq.ZMQError:
                    break
        return out

    # ------------------------------------------------------------------ memory
    def init_memory_pool_and_cache(self):
        from ..mem_cache.registry import TreeCacheBuildContext, create_tree_cache
        rp = getattr(getattr(self.tp_worker, "model_runner", None), "recurrent_pool", None)
        built = create_tree_cache(TreeCacheBuildContext(
            self.server_args, self.model_config, self.req_to_token_pool, self.token_to_kv_pool,
            self.max_total_num_tokens, self.page_size, self.spec_algorithm, rp))
        self.token_to_kv_pool_allocator, self.tree_cache = built.allocator, built.tree_cache
        if built.needs_sequential_schedule:
            self.enable_overlap = False
            self.server_args.disable_overlap_schedule = True

    @property
    def _hicache(self) -> bool:
        return hasattr(self.tree_cache, "check_hicache_events")

    def _empty_batch(self) -> ScheduleBatch:
        return ScheduleBatch([], self.req_to_token_pool, self.token_to_kv_pool_allocator, self.tree_cache,
                             self.vocab_size, self.enable_overlap, self.page_size, self.spec_algorithm)

    # ------------------------------------------------------------------ event loops
    def event_loop_normal(self, stop_event: threading.Event | None = None):
        while not (stop_event is not None and stop_event.is_set()):
            self.step_normal()

    def step_normal(self) -> bool:
        """One iteration without overlap; returns whether a batch ran."""
        self.process_input_requests(self.recv_requests())
        if self._paused:
            time.sleep(0.001)
            return False
        if self._hicache:
            self.tree_cache.check_hicache_events()
        if self.disagg_mode == "prefill":
            self.process_disagg_prefill_inflight()
        elif self.disagg_mode == "decode":
            self.process_disagg_decode_queues()
        batch = self.get_next_batch_to_run()
        self.cur_batch = batch
        if batch is None:
            self.on_idle()
            for h in self.step_hooks:
                h(self, None)
            return False
        result = self.run_batch(batch)
        self.process_batch_result(batch, result)
        self.last_batch = batch
        for h in self.step_hooks:
            h(self, batch)
        return True

    def event_loop_overlap(self, stop_event: threading.Event | None = None):
        while not (stop_event is not None and stop_event.is_set()):
            self.step_overlap()

    def step_overlap(self) -> bool:
        self.process_input_requests(self.recv_requests())
        if self._paused:
            self._drain_results()
            time.sleep(0.001)
            return False
        if self._hicache:
            self.tree_cache.check_hicache_events()
        if self.disagg_mode == "prefill":
            self.process_disagg_prefill_inflight()
        elif self.disagg_mode == "decode":
            self.process_disagg_decode_queues()
        batch = self.get_next_batch_to_run()
        self.cur_batch = batch
        if batch is not None:
            if batch.has_grammar or batch.return_logprob or self.spec_algorithm is not None:
                # these need step n's real tokens before step n+1 can be built
                self._drain_results()
            result = self.run_batch(batch)
            self.result_queue.append((batch.copy(), result))
        if len(self.result_queue) > (1 if batch is not None else 0):
            b, r = self.result_queue.popleft()
            self.process_batch_result(b, r)
        elif batch is None:
            self.on_idle()
        self.last_batch = batch
        for h in self.step_hooks:
            h(self, batch)
        return batch is not None

    def _drain_results(self):
        while self.result_queue:
            b, r = self.result_queue.popleft()
            self.process_batch_result(b, r)

    def on_idle(self):
        self.check_memory()
        self.new_token_ratio = self.init_new_token_ratio
        if self.server_args.sleep_on_idle or self._recv_q is not None:
            time.sleep(0.0005)

    # ------------------------------------------------------------------ requests in
    def process_input_requests(self, reqs: list):
        for r in reqs:
            if isinstance(r, HealthCheckOutput):
                continue
            fn = self._dispatch.get(type(r))
            if fn is None:
                for t, f in self._dispatch.items():
                    if isinstance(r, t):
                        fn = f
                        break
            if fn is None:
                logger.warning("scheduler: unknown message %s", type(r))
                continue
            out = fn(r)
            if out is not None:
                self.send_to_tokenizer(out)
        self.move_ready_grammar_requests()

    def handle_generate_request(self, recv: TokenizedGenerateReqInput):
        sp = recv.sampling_params
        if isinstance(sp, dict):
            sp = SamplingParams.from_dict(sp)
        elif sp is None:
            sp = SamplingParams()
        if not getattr(sp, "stop_strs", None) and sp.stop_strs is None:
            sp.normalize(self.tokenizer)
        extra_key = recv.extra_key
        if recv.mm_inputs and recv.mm_inputs.get("input_embedding") is not None:
            # placeholder tokens look the same for every image / clip: key the prefix cache by the media too
            tag = recv.mm_inputs.get("hash")
            if tag is None:
                import hashlib
                import torch as _t
                emb = _t.as_tensor(recv.mm_inputs["input_embedding"]).detach().cpu().contiguous()
                tag = hashlib.sha1(emb.view(_t.uint8).numpy().tobytes()).hexdigest()[:16]
            extra_key = f"{extra_key or ''}|mm:{tag}"
        req = Req(recv.rid, recv.text, recv.input_ids, sp, return_logprob=bool(recv.return_logprob),
                  top_logprobs_num=recv.top_logprobs_num or 0, token_ids_logprob=recv.token_ids_logprob,
                  stream=recv.stream, lora_id=recv.lora_id, eos_token_ids=self.model_config.hf_eos_token_id,
                  vocab_size=self.vocab_size, extra_key=extra_key, dp_rank=recv.dp_rank,
                  return_hidden_states=recv.return_hidden_states,
                  return_routed_experts=bool(recv.return_routed_experts),
                  return_output_logprob_only=bool(recv.return_output_logprob_only),
                  logprob_start_len=recv.logprob_start_len if recv.logprob_start_len is not None else -1,
                  session_id=recv.session_id, bootstrap_host=recv.bootstrap_host,
                  bootstrap_port=recv.bootstrap_port, bootstrap_room=recv.bootstrap_room,
                  mm_inputs=recv.mm_inputs)
        req.tokenizer = self.tokenizer
        if req.lora_id is not None and not self.server_args.enable_lora:
            return self._reject(req, "LoRA is not enabled on this server (--enable-lora).")
        # ---- length validation
        n_in = len(req.origin_input_ids)
        if n_in >= self.max_req_input_len:
            if self.server_args.allow_auto_truncate:
                req.origin_input_ids = req.origin_input_ids[: self.max_req_input_len]
                req.origin_input_ids_unpadded = req.origin_input_ids
            else:
                return self._reject(req, f"Input length ({n_in} tokens) exceeds the maximum allowed length "
                                         f"({self.max_req_input_len} tokens). Use a shorter input or enable "
                                         f"--allow-auto-truncate.")
        if req.logprob_start_len >= len(req.origin_input_ids) and req.return_logprob:
            return self._reject(req, f"logprob_start_len ({req.logprob_start_len}) is not smaller than the "
                                     f"input length ({len(req.origin_input_ids)}).")
        sp.max_new_tokens = min(sp.max_new_tokens if sp.max_new_tokens is not None else 1 << 30,
                                self.max_req_len - len(req.origin_input_ids) - 1)
        if sp.max_new_tokens < 0:
            sp.max_new_tokens = 0
        # ---- grammar
        if sp.has_grammar:
            if self.grammar_backend is None:
                return self._reject(req, "Grammar-constrained decoding needs a tokenizer "
                                         "(do not use --skip-tokenizer-init).")
            key = next((k, v) for k, v in (("json", sp.json_schema), ("regex", sp.regex), ("ebnf", sp.ebnf),
                                           ("structural_tag", sp.structural_tag)) if v is not None)
            req.grammar_key = key
            val, hit = self.grammar_backend.get_cached_or_future_value(key)
            req.grammar = val
            if not hit:
                self.grammar_queue.append(req)
                return None
            if getattr(val, "is_invalid", False):
                return self._reject(req, f"Invalid grammar request: {key}")
        if self.disagg_mode == "prefill":
            self.disagg_prefill_admit(req)
        elif self.disagg_mode == "decode" and self.disagg_decode_admit(req):
            return None
        self._add_request_to_queue(req)
        return None

    def handle_embedding_request(self, recv: TokenizedEmbeddingReqInput):
        req = Req(recv.rid, recv.text, recv.input_ids, SamplingParams(max_new_tokens=0),
                  vocab_size=self.vocab_size, extra_key=recv.extra_key)
        req.is_embedding_req = True
        if len(req.origin_input_ids) >= self.max_req_input_len:
            return self._reject(req, "Input length exceeds the maximum allowed length.")
        self._add_request_to_queue(req)

    def _reject(self, req: Req, message: str):
        """Finish a request that never ran, through the normal output path."""
        req.finished_reason = FINISH_ABORT(message, 400, "BadRequestError")
        req.origin_input_ids = req.origin_input_ids[:1] or [0]
        self.stream_output([req], False)
        return None

    def _add_request_to_queue(self, req: Req):
        req.queue_time_start = time.perf_counter()
        self.waiting_queue.append(req)

    def move_ready_grammar_requests(self):
        """Requests waiting for an asynchronous grammar compile join the queue once it is done
        (reference :1422-1467); compiles that take too long abort the request."""
        if not self.grammar_queue:
            return
        still = []
        for req in self.grammar_queue:
            fut = req.grammar
            if hasattr(fut, "done") and not fut.done():
                req.grammar_wait_ct += 1
                if req.grammar_wait_ct > 300_000:
                    self._reject(req, "Grammar compilation timed out.")
                else:
                    still.append(req)
                continue
            val = fut.result() if hasattr(fut, "result") else fut
            self.grammar_backend.set_cache(req.grammar_key, val)
            if getattr(val, "is_invalid", False):
                self._reject(req, f"Invalid grammar request: {getattr(val, 'error', req.grammar_key)}")
                continue
            req.grammar = val.copy() if hasattr(val, "copy") else val
            self._add_request_to_queue(req)
        self.grammar_queue = still

    # ------------------------------------------------------------------ batch selection
    def get_next_batch_to_run(self) -> ScheduleBatch | None:
        # fold the previous prefill into the running decode batch
        if self.last_batch is not None and self.last_batch.forward_mode is not None and \
                self.last_batch.forward_mode.is_extend():
            lb = self.last_batch
            if self.chunked_req is not None and self.chunked_req in lb.reqs:
                # publish what has been prefilled so far; the request keeps its row
                self.tree_cache.cache_unfinished_req(self.chunked_req, chunked=True)
            if lb.decoding_reqs:
                # mixed step: the decode rows already live in running_batch
                keep = [i for i, r in enumerate(lb.reqs) if r not in lb.decoding_reqs]
                lb.filter_batch(keep_indices=keep)
            lb.filter_batch(chunked_req_to_exclude=self.chunked_req)
            if not lb.is_empty() and not self.is_embedding:
                if self.running_batch.is_empty():
                    self.running_batch = lb
                else:
                    self.running_batch.merge_batch(lb)
            self.last_batch = None

        force_decode = (self.decode_first_interleave > 0 and not self.running_batch.is_empty()
                        and self.decode_steps_since_prefill < self.decode_first_interleave)
        new_batch = None if force_decode else self.get_new_batch_prefill()
        if new_batch is not None:
            self.decode_steps_since_prefill = 0
            return new_batch
        if self.running_batch.is_empty():
            return None
        self.running_batch = self.update_running_batch(self.running_batch)
        self.decode_steps_since_prefill += 1
        return self.running_batch if not self.running_batch.is_empty() else None

    def get_new_batch_prefill(self) -> ScheduleBatch | None:
        if (self.running_batch.batch_is_full or not self.waiting_queue) and self.chunked_req is None:
            return None
        # rows of requests that have just finished are free again (they leave the batch at its next filter)
        running_bs = sum(1 for r in self.running_batch.reqs if not r.finished())
        if running_bs >= self.max_running_requests and self.chunked_req is None:
            self.running_batch.batch_is_full = True
            return None
        if TEST_RETRACT and running_bs > TEST_RETRACT_NO_PREFILL_BS:
            return None
        self.policy.calc_priority(self.waiting_queue)
        mixed = self.server_args.enable_mixed_chunk and not self.running_batch.is_empty() \
            and not self.running_batch.return_logprob
        adder = PrefillAdder(self.page_size, self.tree_cache, self.token_to_kv_pool_allocator, self.running_batch,
                             self.new_token_ratio, self.max_prefill_tokens, self.chunked_prefill_size,
                             running_bs if mixed else 0)
        if self.chunked_req is not None:
            self.chunked_req.init_next_round_input(None)
            self.chunked_req = adder.add_chunked_req(self.chunked_req)

        # adapters of one batch must fit the LoRA slots (reference `scheduler.py` lora_set check)
        lora_set = None
        if self.server_args.enable_lora:
            lora_set = {r.lora_id for r in self.running_batch.reqs if r.lora_id is not None}
            if self.chunked_req is not None and self.chunked_req.lora_id is not None:
                lora_set.add(self.chunked_req.lora_id)

        for req in list(self.waiting_queue):
            if running_bs + len(adder.can_run_list) >= self.max_running_requests:
                self.running_batch.batch_is_full = True
                break
            if self.req_to_token_pool.available_size() - len([r for r in adder.can_run_list if r.req_pool_idx is None]) <= 0:
                self.running_batch.batch_is_full = True
                break
            if adder.new_chunked_req is not None:
                break   # one request is chunked per step; the rest of its budget is spent
            if lora_set is not None and req.lora_id is not None and req.lora_id not in lora_set:
                if len(lora_set) >= self.server_args.max_loras_per_batch:
                    continue      # would exceed the adapters one batch can hold; try a later request
            req.init_next_round_input(self.tree_cache)
            res = adder.add_one_req(req)
            if lora_set is not None and res == AddReqResult.CONTINUE and req.lora_id is not None:
                lora_set.add(req.lora_id)
            if res != AddReqResult.CONTINUE:
                if res == AddReqResult.NO_TOKEN:
                    self.running_batch.batch_is_full = True
                break

        can_run = adder.can_run_list
        if not can_run:
            return None
        run_set = set(id(r) for r in can_run)
        self.waiting_queue = [r for r in self.waiting_queue if id(r) not in run_set]
        if adder.new_chunked_req is not None:
            assert self.chunked_req is None
            self.chunked_req = adder.new_chunked_req
        if self.chunked_req is not None:
            self.chunked_req.is_chunked += 1
        for r in can_run:
            if r.queue_time_end is None:
                r.queue_time_end = time.perf_counter()
        self.log_prefill_stats(adder, can_run, running_bs)

        batch = ScheduleBatch.init_new(can_run, self.req_to_token_pool, self.token_to_kv_pool_allocator,
                                       self.tree_cache, self.vocab_size, self.enable_overlap, self.page_size,
                                       self.spec_algorithm, self.chunked_req)
        batch.prepare_for_extend()
        if mixed and not batch.return_logprob:
            self.running_batch.filter_batch()
            if not self.running_batch.is_empty():
                batch.mix_with_running(self.running_batch)
        return batch

    def update_running_batch(self, batch: ScheduleBatch) -> ScheduleBatch:
        batch.filter_batch()
        if self.draft_worker is not None:
            batch.spec_alloc_len = self.draft_worker.alloc_len
        if batch.is_empty():
            batch.batch_is_full = False
            return batch
        forced = TEST_RETRACT and self.forward_ct % TEST_RETRACT_INTERVAL == 0 and len(batch.reqs) > 1
        if forced or not batch.check_decode_mem():
            old_ratio = self.new_token_ratio
            if self.enable_overlap:
                self._drain_results()   # retraction needs the requests' real state
                batch.filter_batch()
                if batch.is_empty():
                    return batch
            retracted, new_ratio, aborted = batch.retract_decode(self.server_args)
            self.total_retracted_reqs += len(retracted)
            self.new_token_ratio = new_ratio
            logger.info("KV cache pool is full. Retract requests. #retracted_reqs: %d, #aborted: %d, "
                        "#new_token_ratio: %.4f -> %.4f", len(retracted), len(aborted), old_ratio, new_ratio)
            for r in retracted:
                self._add_request_to_queue(r)
            if aborted:
                self.stream_output(aborted, False)
        else:
            self.new_token_ratio = max(self.new_token_ratio - self.new_token_ratio_decay, self.min_new_token_ratio)
        if batch.is_empty():
            return batch
        if batch.batch_is_full and len(batch.reqs) < self.max_running_requests:
            batch.batch_is_full = False
        batch.prepare_for_decode()
        return batch

    # ------------------------------------------------------------------ run
    def run_batch(self, batch: ScheduleBatch):
        self.forward_ct += 1
        if self._hicache:
            # pages being loaded back from the host tier must land before this batch reads them
            self.tree_cache.ready_to_load_host_cache()
        self._profile_batch_predicate(batch)
        if self.is_embedding:
            mwb = batch.get_model_worker_batch()
            return SimpleNamespace(embeddings=self.tp_worker.forward_batch_embedding(mwb), next_token_ids=None,
                                   logits_output=None)
        if self.draft_worker is not None:
            return self.draft_worker.forward_batch_speculative_generation(batch)
        mwb = batch.get_model_worker_batch()
        if self.enable_overlap:
            mwb.future_slots = (mwb.req_pool_indices.astype(np.int64) + 1)
            if mwb.forward_mode.is_extend():
                # rows of non-final chunks produce no token; park their sample in the spare slot 0
                # (`is_chunked` lags one step in overlap mode; `batch.chunked_req` is exact)
                chunk_rows = np.array([r is batch.chunked_req for r in batch.reqs])
                mwb.future_slots = np.where(chunk_rows, 0, mwb.future_slots)
        if batch.has_grammar:
            self._fill_vocab_mask(batch, mwb)
        return self.tp_worker.forward_batch_generation(mwb)

    def _fill_vocab_mask(self, batch: ScheduleBatch, mwb):
        words = (self.vocab_size + 31) // 32
        mask = np.full((len(batch.reqs), words), -1, dtype=np.int32)
        for i, r in enumerate(batch.reqs):
            if r.grammar is not None and not r.finished():
                r.grammar.fill_vocab_mask(mask, i)
        mwb.sampling_info.vocab_mask = mask
        mwb.sampling_info.is_all_greedy = mwb.sampling_info.is_all_greedy

    def process_batch_result(self, batch: ScheduleBatch, result):
        if self.is_embedding:
            self.process_batch_result_embedding(batch, result.embeddings)
        elif batch.forward_mode.is_decode():
            if getattr(result, "spec_tokens", None) is not None:
                self.process_batch_result_spec_decode(batch, result)
            else:
                self.process_batch_result_decode(batch, result)
        elif batch.forward_mode.is_extend():
            self.process_batch_result_prefill(batch, result)
        self.watchdog_last_forward_ct = self.forward_ct

    # ------------------------------------------------------------------ control
    def abort_request(self, recv: AbortReq):
        """Reference :2749-2857: waiting requests finish immediately; running ones are flagged
        and finish at their next result; a request in the middle of chunked prefill is dropped
        with its KV."""
        def match(r: Req) -> bool:
            return recv.abort_all or r.rid == recv.rid or (isinstance(recv.rid, str) and r.rid.startswith(recv.rid))

        msg = recv.aborted_message or "Aborted by the client."
        hit, keep = [], []
        for r in self.waiting_queue:
            (hit if match(r) else keep).append(r)
        self.waiting_queue = keep
        for r in hit:
            r.finished_reason = FINISH_ABORT(msg)
            if r.req_pool_idx is not None:      # was retracted / chunked and owns nothing now
                self.req_to_token_pool.free(r.req_pool_idx)
                r.req_pool_idx = None
        if hit:
            self.stream_output(hit, False)
        if self.disagg_mode == "decode":
            pq = self.disagg_prealloc_queue
            for r in [r for r in pq.queue if match(r)]:
                pq.queue.remove(r)
                r.finished_reason = FINISH_ABORT(msg)
                self.stream_output([r], False)
            for r in self.disagg_transfer_queue.queue:
                if match(r):
                    r.to_abort, r.to_abort_message = True, msg
        gq = [r for r in self.grammar_queue if match(r)]
        self.grammar_queue = [r for r in self.grammar_queue if not match(r)]
        for r in gq:
            self._reject(r, msg)
        if self.chunked_req is not None and match(self.chunked_req):
            self._drain_results()
            r = self.chunked_req
            self.chunked_req = None
            r.finished_reason = FINISH_ABORT(msg)
            r.is_chunked = 0
            tmp = self._empty_batch()
            tmp._release_req(r)
            r.req_pool_idx = None
            if self.last_batch is not None and r in self.last_batch.reqs:
                self.last_batch.filter_batch()
            self.stream_output([r], False)
        for r in self.running_batch.reqs:
            if match(r) and not r.finished():
                r.to_abort = True
                r.to_abort_message = msg
        if self.last_batch is not None:
            for r in self.last_batch.reqs:
                if match(r) and not r.finished():
                    r.to_abort = True
                    r.to_abort_message = msg
        return None

    def pause_generation(self, recv: PauseGenerationReqInput):
        """Reference :2859-2907."""
        self._drain_results()
        self._paused = True
        if recv.mode == "abort":
            self.abort_request(AbortReq(abort_all=True, aborted_message="Aborted by pause_generation."))
            # flagged running requests finish without another forward
            self._fold_last_batch()
            for r in list(self.running_batch.reqs):
                if not r.finished():
                    r.check_finished()
                    if r.finished():
                        self._finish_req(r)
            self.stream_output(self.running_batch.reqs, False)
            self.running_batch.filter_batch()
        elif recv.mode == "retract":
            self._fold_last_batch()
            rb = self.running_batch
            for r in list(rb.reqs):
                if not r.finished():
                    rb._release_req(r)
                    r.reset_for_retract()
                    self._add_request_to_queue(r)
            self.running_batch = self._empty_batch()
            if self.chunked_req is not None:
                r = self.chunked_req
                self.chunked_req = None
                tmp = self._empty_batch()
                tmp._release_req(r)
                r.reset_for_retract()
                self.waiting_queue.insert(0, r)
        return None

    def _fold_last_batch(self):
        lb = self.last_batch
        if lb is not None and lb.forward_mode is not None and lb.forward_mode.is_extend():
            if self.chunked_req is not None and self.chunked_req in lb.reqs:
                self.tree_cache.cache_unfinished_req(self.chunked_req, chunked=True)
            lb.filter_batch(chunked_req_to_exclude=self.chunked_req)
            if lb.decoding_reqs:
                lb.filter_batch(keep_indices=[i for i, r in enumerate(lb.reqs) if r not in lb.decoding_reqs])
            if not lb.is_empty():
                if self.running_batch.is_empty():
                    self.running_batch = lb
                else:
                    self.running_batch.merge_batch(lb)
        self.last_batch = None

    def continue_generation(self, recv: ContinueGenerationReqInput):
        self._paused = False
        return None

    # ------------------------------------------------------------------ LoRA
    def load_lora_adapter(self, recv: LoadLoRAAdapterReqInput) -> LoRAUpdateOutput:
        ok, msg = self.tp_worker.load_lora_adapter(recv)
        return LoRAUpdateOutput(request_id=recv.request_id, success=ok, error_msg=msg)

    def unload_lora_adapter(self, recv: UnloadLoRAAdapterReqInput) -> LoRAUpdateOutput:
        ok, msg = self.tp_worker.unload_lora_adapter(recv)
        return LoRAUpdateOutput(request_id=recv.request_id, success=ok, error_msg=msg)

    def flush_cache_wrapped(self, recv: FlushCacheReqInput):
        ok, n = self.flush_cache()
        return FlushCacheReqOutput(success=ok, flushed_items=n,
                                   error_msg="" if ok else "Cache not flushed because there are pending requests.")

    def flush_cache(self) -> tuple[bool, int]:
        self._drain_results()
        self._fold_last_batch()
        self.running_batch.filter_batch()
        if self.waiting_queue or not self.running_batch.is_empty() or self.chunked_req is not None:
            logger.warning("Cache not flushed because there are pending requests. #queue-req: %d, #running-req: %d",
                           len(self.waiting_queue), len(self.running_batch.reqs))
            return False, 0
        n = self.tree_cache.total_size() if hasattr(self.tree_cache, "total_size") else 0
        self.cur_batch = None
        self.last_batch = None
        self.tree_cache.reset()
        self.req_to_token_pool.clear()
        self.token_to_kv_pool_allocator.clear()
        self.tp_worker.flush()
        if self.grammar_backend is not None:
            self.grammar_backend.reset()
        self.new_token_ratio = self.init_new_token_ratio
        logger.info("Cache flushed successfully!")
        return True, n

    def get_internal_state(self, recv: GetInternalStateReq):
        used, usage = self.token_usage()
        st = dict(self.server_args.to_dict())
        st.update({
            "last_gen_throughput": self.last_gen_throughput,
            "max_total_num_tokens": self.max_total_num_tokens,
            "max_running_requests": self.max_running_requests,
            "max_req_input_len": self.max_req_input_len,
            "token_usage": usage,
            "num_running_reqs": len(self.running_batch.reqs),
            "num_waiting_reqs": len(self.waiting_queue),
            "total_retracted_reqs": self.total_retracted_reqs,
            "forward_ct": self.forward_ct,
            "cuda_graph_recaptures": self.graph_recapture_count(),
            "cuda_graph_replays": getattr(getattr(self.tp_worker, "model_runner", None), "graph_replays", 0),
            "precision_tracer": dict(self.precision_tracer_state),
        })
        if self.spec_algorithm is not None and self.spec_num_total_forward_ct:
            st["avg_spec_accept_length"] = self.spec_num_total_accepted_tokens / self.spec_num_total_forward_ct
        return GetInternalStateReqOutput(st)

    def set_internal_state(self, recv: SetInternalStateReq):
        """Reference :1533-1590: a small set of runtime-settable knobs (and the precision tracer)."""
        ok = True
        for k, v in recv.state_data.items():
            if k == "precision_tracer":
                self.precision_tracer_state.update(v)
                from ..utils.precision_tracer import precision_tracer
                precision_tracer.apply_state(self.precision_tracer_state)
            elif k in ("max_micro_batch_size", "stream_interval", "decode_log_interval",
                       "schedule_conservativeness", "chunked_prefill_size", "max_prefill_tokens"):
                setattr(self.server_args, k, v)
                if k == "stream_interval":
                    self.stream_interval = v
                if k == "chunked_prefill_size":
                    self.chunked_prefill_size = v if v and v > 0 else None
                if k == "max_prefill_tokens":
                    self.max_prefill_tokens = v
            else:
                ok = False
        return SetInternalStateReqOutput(recv.request_id, ok, "" if ok else "unknown key", ok,
                                         self.server_args.to_dict())

    def open_session(self, recv: OpenSessionReqInput):
        if recv.session_id in self.sessions:
            return OpenSessionReqOutput(recv.request_id, False, "session exists", recv.session_id)
        self.sessions[recv.session_id] = {"created": time.time()}
        return OpenSessionReqOutput(recv.request_id, True, "", recv.session_id)

    def close_session(self, recv: CloseSessionReqInput):
        ok = self.sessions.pop(recv.session_id, None) is not None
        return CloseSessionReqOutput(recv.request_id, ok, "" if ok else "unknown session")

    def configure_logging(self, recv: ConfigureLoggingReq):
        if recv.log_level:
            logging.getLogger().setLevel(recv.log_level.upper())
        return ConfigureLoggingReqOutput(recv.request_id)

    def graph_recapture_count(self) -> int:
        mr = getattr(self.tp_worker, "model_runner", None)
        return getattr(mr, "graph_recaptures", 0) if mr is not None else 0

    # ------------------------------------------------------------------ invariants / watchdog
    def check_memory(self):
        """Leak invariant on idle (reference :1723-1775): every slot is either free, held by an
        evictable tree node, or protected by a lock that some request still holds."""
        if self.chunked_req is not None or self.result_queue:
            return
        if self.disagg_mode == "prefill" and self.disagg_prefill_inflight:
            return
        if self.disagg_mode == "decode" and (self.disagg_prealloc_queue.queue or self.disagg_transfer_queue.queue):
            return
        if not self.running_batch.is_empty() or self.waiting_queue and any(r.req_pool_idx is not None for r in self.waiting_queue):
            return
        pool = getattr(getattr(self.tp_worker, "model_runner", None), "token_to_kv_pool", None)
        if getattr(pool, "check_canaries", None) is not None:
            pool.check_canaries()          # guard pages behind the KV buffers (SGLB_KV_CANARY_PAGES), untouched?
        if hasattr(self.tree_cache, "swa_evictable_size"):
            # hybrid sliding-window pools: the invariant holds for each pool separately
            al, tc = self.token_to_kv_pool_allocator, self.tree_cache
            ps_ = self.page_size
            for name, avail, ev, prot, size in (
                    ("full", al.full_available_size(), tc.full_evictable_size(), tc.full_protected_size(), al.size),
                    ("swa", al.swa_available_size(), tc.swa_evictable_size(), tc.swa_protected_size(), al.size_swa)):
                if avail + ev + prot != size // ps_ * ps_ or prot != 0:
                    msg = (f"KV cache pool leak detected ({name})! available={avail} evictable={ev} "
                           f"protected={prot} expected={size // ps_ * ps_}")
                    logger.error(msg)
                    if os.environ.get("SGLANG_STRICT_MEMORY_CHECK", "1") == "1":
                        raise RuntimeError(msg)
            return
        avail = self.token_to_kv_pool_allocator.available_size()
        evictable = self.tree_cache.evictable_size()
        protected = self.tree_cache.protected_size()
        total = avail + evictable + protected
        expect = self.max_total_num_tokens if self.page_size == 1 else \
            self.max_total_num_tokens // self.page_size * self.page_size
        if total != expect or protected != 0:
            msg = (f"KV cache pool leak detected! available={avail} evictable={evictable} protected={protected} "
                   f"total={total} expected={expect}")
            logger.error(msg)
            if os.environ.get("SGLANG_STRICT_MEMORY_CHECK", "1") == "1":
                raise RuntimeError(msg)
        free_rows = self.req_to_token_pool.available_size()
        if free_rows != self.req_to_token_pool.size and not self.waiting_queue:
            msg = f"req_to_token_pool leak detected! free={free_rows} size={self.req_to_token_pool.size}"
            logger.error(msg)
            if os.environ.get("SGLANG_STRICT_MEMORY_CHECK", "1") == "1":
                raise RuntimeError(msg)

    def watchdog_thread(self):
        """Kills the server if a batch has been in flight for `watchdog_timeout` seconds without
        any forward step completing (reference :2724-2747)."""
        timeout = self.server_args.watchdog_timeout
        last_ct, last_t = self.forward_ct, time.perf_counter()
        while not self._watchdog_stop.wait(min(timeout / 2, 5.0)):
            now = time.perf_counter()
            if self.cur_batch is not None and self.forward_ct == last_ct:
                if now - last_t > timeout:
                    logger.error("Scheduler watchdog timeout (%.0fs without progress); dumping stacks", timeout)
                    faulthandler.dump_traceback()
                    try:
                        os.kill(self.parent_pid, signal.SIGQUIT)
                    finally:
                        os._exit(1)
            else:
                last_ct, last_t = self.forward_ct, now

    def shutdown(self):
        self._watchdog_stop.set()
        try:
            self.tp_worker.shutdown()
        except Exception:
            pass


def run_scheduler_process(server_args, port_args, pipe_writer=None, rank: int = 0, world_size: int = 1,
                          init_method: str | None = None):
    """Entry of the scheduler subprocess (tensor rank 0) and of follower ranks."""
    from ..parallel import state as ps
    from ..utils.common import configure_logger, kill_itself_when_parent_died
    faulthandler.enable()
    kill_itself_when_parent_died()
    configure_logger(server_args, prefix=f" TP{rank}")
    try:
        local = rank % max(world_size // max(server_args.nnodes, 1), 1)
        if server_args.device_indexes:
            local = server_args.device_indexes[local]
        dp = server_args.dp_size if world_size > 1 else 1
        ps.init_distributed(rank, world_size, server_args.device, dp, server_args.ep_size,
                            init_method=init_method, local_rank=local, timeout_s=server_args.dist_timeout)
        if rank != 0:
            from .tp_worker import run_tp_follower
            if pipe_writer is not None:
                pipe_writer.send({"status": "ready"})
            if dp > 1 and rank % (world_size // dp) == 0:
                # first rank of a data-parallel section: executes that section's batches for the one scheduler
                from .dp_scheduler import run_dp_leader
                run_dp_leader(server_args)
            else:
                run_tp_follower(server_args)
            return
        if dp > 1:
            from .dp_scheduler import DPScheduler, connect_sections
            from .tp_worker import ModelWorker
            assert server_args.speculative_algorithm is None and server_args.disaggregation_mode in (None, "null"), \
                "data-parallel attention runs without speculative decoding and without PD disaggregation"
            sched = DPScheduler(server_args, port_args, connect_sections(server_args, ModelWorker(server_args)))
        else:
            sched = Scheduler(server_args, port_args)
        if pipe_writer is not None:
            pipe_writer.send({"status": "ready", "max_total_num_tokens": sched.max_total_num_tokens,
                              "max_req_input_len": sched.max_req_input_len})
        if sched.enable_overlap:
            sched.event_loop_overlap()
        else:
            sched.event_loop_normal()
    except Exception:
        import traceback
        logger.error("Scheduler hit an exception: %s", traceback.format_exc())
        try:
            os.kill(os.getppid(), signal.SIGQUIT)
        except Exception:
            pass
        raise
