"""Front-end manager: tokenises requests, forwards them to the scheduler, collects the
streamed outputs and exposes the control RPCs.

Reference: `python/sgl_jax/srt/managers/tokenizer_manager.py:117-1503` (`generate_request` :254,
`_tokenize_one_request` :293, `_create_tokenized_object` :345, client-disconnect abort :555,
batch fan-out and the `n > 1` prefix-cache trick :621-700, request logging levels :847-892,
crash dump :956, `handle_loop` :1044, `convert_logprob_style` :1165, `score_request` :1347,
`_Communicator` :1468).
"""

from __future__ import annotations

import asyncio
import copy
import dataclasses
import json
import logging
import os
import queue
import threading
import time
import uuid
from typing import Any, AsyncGenerator

from ..sampling.sampling_params import SamplingParams
from .io_struct import (AbortReq, BatchEmbeddingOut, BatchStrOut, CloseSessionReqInput, ConfigureLoggingReq,
                        ContinueGenerationReqInput, EmbeddingReqInput, FlushCacheReqInput, FlushCacheReqOutput, LoadLoRAAdapterReqInput,
                        LoRAUpdateOutput, SchedulerFailure, UnloadLoRAAdapterReqInput,
                        GenerateReqInput, GetInternalStateReq, GetInternalStateReqOutput, GetLoadReqInput,
                        GetLoadReqOutput, OpenSessionReqInput, PauseGenerationReqInput, ProfileReq,
                        ProfileReqOutput, ProfileReqType, SetInternalStateReq, SetInternalStateReqOutput,
                        TokenizedEmbeddingReqInput, TokenizedGenerateReqInput)

logger = logging.getLogger(__name__)


@dataclasses.dataclass
class ReqState:
    out_list: list
    finished: bool
    event: asyncio.Event
    obj: Any
    created_time: float
    lora_id: Any = None
    first_token_time: float = 0.0
    finished_time: float = 0.0
    last_output_offset: int = 0
    text: str = ""
    output_ids: list = dataclasses.field(default_factory=list)
    input_token_logprobs: list = dataclasses.field(default_factory=list)
    output_token_logprobs: list = dataclasses.field(default_factory=list)
    input_top_logprobs: list = dataclasses.field(default_factory=list)
    output_top_logprobs: list = dataclasses.field(default_factory=list)
    input_token_ids_logprobs: list = dataclasses.field(default_factory=list)
    output_token_ids_logprobs: list = dataclasses.field(default_factory=list)


class _Communicator:
    """One outstanding RPC of a kind: send a request object, await `fan_out` replies."""

    def __init__(self, sender, fan_out: int = 1):
        self._sender = sender
        self._fan_out = fan_out
        self._event: asyncio.Event | None = None
        self._values: list | None = None
        self._lock = asyncio.Lock()

    async def __call__(self, obj, timeout: float | None = 120.0):
        async with self._lock:
            self._event = asyncio.Event()
            self._values = []
            self._sender.send_pyobj(obj)
            await asyncio.wait_for(self._event.wait(), timeout)
            vals, self._values, self._event = self._values, None, None
            return vals

    def handle_recv(self, obj):
        if self._values is None:
            return
        self._values.append(obj)
        if len(self._values) >= self._fan_out:
            self._event.set()


class TokenizerManager:
    def __init__(self, server_args, port_args=None, send_to_scheduler=None, recv_from_detokenizer=None,
                 tokenizer=None, model_config=None):
        self.server_args = server_args
        self.port_args = port_args
        self.enable_metrics = server_args.enable_metrics
        self.log_requests = server_args.log_requests
        self.log_requests_level = server_args.log_requests_level
        self.crash_dump_folder = server_args.crash_dump_folder
        self.crash_dump_request_list: list = []
        self.send_to_scheduler = send_to_scheduler
        self.recv_from_detokenizer = recv_from_detokenizer
        if send_to_scheduler is None and port_args is not None:
            import zmq
            import zmq.asyncio
            from .communication import get_zmq_socket
            ctx = zmq.asyncio.Context(2)
            self.recv_from_detokenizer = get_zmq_socket(ctx, zmq.PULL, port_args.tokenizer_ipc_name, True)
            sctx = zmq.Context(1)
            self.send_to_scheduler = get_zmq_socket(sctx, zmq.PUSH, port_args.scheduler_input_ipc_name, False)
        if model_config is None:
            from ..configs.model_config import ModelConfig
            model_config = ModelConfig.from_server_args(server_args)
        self.model_config = model_config
        self.context_len = model_config.context_len
        self.is_generation = not model_config.is_embedding
        self.model_path = server_args.model_path
        self.served_model_name = server_args.served_model_name
        self.tokenizer = tokenizer
        if tokenizer is None and not server_args.skip_tokenizer_init:
            from ..utils.hf_transformers_utils import get_tokenizer
            self.tokenizer = get_tokenizer(server_args.tokenizer_path, server_args.tokenizer_mode,
                                           server_args.trust_remote_code, server_args.revision,
                                           server_args.tokenizer_backend)
        self.preferred_sampling_params = json.loads(server_args.preferred_sampling_params) \
            if server_args.preferred_sampling_params else None
        self.rid_to_state: dict[str, ReqState] = {}
        self.to_create_loop = True
        self.loop: asyncio.AbstractEventLoop | None = None
        self.gracefully_exit = False
        self.last_receive_tstamp = 0.0
        self.max_req_input_len: int | None = None
        self.is_pause = False
        self.is_pause_cond: asyncio.Condition | None = None
        self.session_futures: dict = {}
        self.lora_registry = None
        if server_args.enable_lora:
            from ..lora.lora_registry import LoRARegistry
            self.lora_registry = LoRARegistry(server_args.lora_paths)
        self.lora_update_lock: asyncio.Lock | None = None
        self.cache_miss_count = 0
        self.fatal_error: str | None = None

        s = self.send_to_scheduler
        self.flush_cache_communicator = _Communicator(s)
        self.get_internal_state_communicator = _Communicator(s)
        self.set_internal_state_communicator = _Communicator(s)
        self.profile_communicator = _Communicator(s)
        self.get_load_communicator = _Communicator(s)
        self.session_communicator = _Communicator(s)
        self.generic_communicator = _Communicator(s)
        self.lora_communicator = _Communicator(s)
        self._result_dispatch = {
            FlushCacheReqOutput: self.flush_cache_communicator.handle_recv,
            GetInternalStateReqOutput: self.get_internal_state_communicator.handle_recv,
            SetInternalStateReqOutput: self.set_internal_state_communicator.handle_recv,
            ProfileReqOutput: self.profile_communicator.handle_recv,
            GetLoadReqOutput: self.get_load_communicator.handle_recv,
            LoRAUpdateOutput: self.lora_communicator.handle_recv,
        }
        self.metrics_collector = None
        if self.enable_metrics:
            from ..utils.metrics import TokenizerMetricsCollector
            self.metrics_collector = TokenizerMetricsCollector(server_args)

    # ------------------------------------------------------------------ public: generate
    async def generate_request(self, obj: GenerateReqInput | EmbeddingReqInput, request=None
                               ) -> AsyncGenerator[dict, None]:
        created = time.time()
        self.auto_create_handle_loop()
        obj.normalize_batch_and_arguments()
        if self.log_requests:
            logger.info("Receive: obj=%s", self._fmt_obj(obj))
        if self.is_pause_cond is not None:
            async with self.is_pause_cond:
                await self.is_pause_cond.wait_for(lambda: not self.is_pause)
        if obj.is_single:
            tokenized = await self._tokenize_one_request(obj)
            state = self._send_one_request(obj, tokenized, created)
            async for resp in self._wait_one_response(obj, state, request):
                yield resp
        else:
            async for resp in self._handle_batch_request(obj, request, created):
                yield resp

    async def _tokenize_one_request(self, obj):
        input_ids = obj.input_ids
        text = obj.text
        if input_ids is None:
            if self.tokenizer is None:
                raise ValueError("The engine was initialised with skip_tokenizer_init=True: pass input_ids, not text.")
            input_ids = self.tokenizer.encode(text)
        return self._create_tokenized_object(obj, text, list(input_ids))

    def _batch_tokenize(self, subs: list):
        """`--enable-tokenizer-batch-encode` (reference `tokenizer_manager.py:493`, `:632`): the texts of a batch
        request go through the tokenizer in one call; requests that carry token ids, embeddings or media cannot."""
        if self.tokenizer is None:
            raise ValueError("The engine was initialised with skip_tokenizer_init=True: pass input_ids, not text.")
        for sub in subs:
            if getattr(sub, "input_ids", None) is not None:
                raise ValueError("Batch tokenization is not needed for pre-tokenized input_ids. "
                                 "Do not set `enable_tokenizer_batch_encode`.")
            if getattr(sub, "input_embeds", None) is not None:
                raise ValueError("Batch tokenization is not needed for input_embeds. "
                                 "Do not set `enable_tokenizer_batch_encode`.")
            if getattr(sub, "image_data", None) or getattr(sub, "audio_data", None) or getattr(sub, "video_data", None):
                raise ValueError("For multimodal input processing do not set `enable_tokenizer_batch_encode`.")
        texts = [sub.text for sub in subs]
        enc = self.tokenizer(texts)["input_ids"] if callable(self.tokenizer) else [self.tokenizer.encode(t) for t in texts]
        return [self._create_tokenized_object(sub, sub.text, list(ids)) for sub, ids in zip(subs, enc)]

    def _validate_len(self, obj, n_in: int, sp: SamplingParams | None):
        if self.max_req_input_len is not None and n_in >= self.max_req_input_len and not self.server_args.allow_auto_truncate:
            raise ValueError(f"The input ({n_in} tokens) is longer than the model's context length "
                             f"({self.context_len} tokens).")
        if n_in >= self.context_len and not self.server_args.allow_auto_truncate:
            raise ValueError(f"The input ({n_in} tokens) is longer than the model's context length "
                             f"({self.context_len} tokens).")
        if sp is not None and sp.max_new_tokens is not None and n_in + sp.max_new_tokens >= self.context_len \
                and not self.server_args.allow_auto_truncate:
            raise ValueError(f"Requested token count exceeds the model's maximum context length of "
                             f"{self.context_len} tokens. You requested a total of {n_in + sp.max_new_tokens} tokens: "
                             f"{n_in} tokens from the input messages and {sp.max_new_tokens} tokens for the completion.")

    def _create_tokenized_object(self, obj, text, input_ids):
        if isinstance(obj, EmbeddingReqInput):
            self._validate_len(obj, len(input_ids), None)
            return TokenizedEmbeddingReqInput(obj.rid, text or "", input_ids, obj.normalize, obj.extra_key)
        spd = dict(obj.sampling_params or {})
        if self.preferred_sampling_params:
            spd = {**self.preferred_sampling_params, **spd}
        sp = SamplingParams.from_dict(spd)
        sp.normalize(self.tokenizer)
        sp.verify(self.model_config.vocab_size)
        self._validate_len(obj, len(input_ids), sp)
        lora_id = obj.lora_id
        if self.lora_registry is not None and getattr(self.server_args, "enable_static_lora", False) \
                and self.lora_registry._by_name:
            # `--enable-static-lora`: the first loaded adapter serves every request, whatever the request names
            # (reference `schedule_batch.py:2685`: all rows carry adapter "0")
            obj.lora_path = next(iter(self.lora_registry._by_name))
        if obj.lora_path is not None and self.lora_registry is not None:
            lora_id = self.lora_registry.acquire(obj.lora_path)
        return TokenizedGenerateReqInput(
            rid=obj.rid, text=text, input_ids=input_ids, sampling_params=sp,
            return_logprob=bool(obj.return_logprob), return_output_logprob_only=obj.return_output_logprob_only,
            logprob_start_len=obj.logprob_start_len if obj.logprob_start_len is not None else -1,
            top_logprobs_num=obj.top_logprobs_num or 0, token_ids_logprob=obj.token_ids_logprob,
            stream=obj.stream, lora_id=lora_id, extra_key=obj.extra_key,
            return_routed_experts=bool(obj.return_routed_experts), return_hidden_states=obj.return_hidden_states,
            dp_rank=obj.dp_rank, bootstrap_host=obj.bootstrap_host, bootstrap_port=obj.bootstrap_port,
            bootstrap_room=obj.bootstrap_room, disagg_prefill_dp_rank=obj.disagg_prefill_dp_rank,
            disagg_transfer_id=obj.disagg_transfer_id, mm_inputs=obj.mm_inputs)

    def _send_one_request(self, obj, tokenized, created) -> ReqState:
        state = ReqState([], False, asyncio.Event(), obj, created)
        state.lora_id = getattr(tokenized, "lora_id", None)
        self.rid_to_state[obj.rid] = state
        self.send_to_scheduler.send_pyobj(tokenized)
        return state

    async def _wait_one_response(self, obj, state: ReqState, request=None):
        while True:
            try:
                await asyncio.wait_for(state.event.wait(), timeout=4)
            except asyncio.TimeoutError:
                if request is not None and await request.is_disconnected():
                    self.abort_request(obj.rid)
                    raise ValueError(f"Request is disconnected from the client side. Abort request rid={obj.rid}")
                continue
            if self.fatal_error is not None and not state.out_list:
                self.rid_to_state.pop(obj.rid, None)
                raise RuntimeError(f"scheduler failure: {self.fatal_error}")
            out = state.out_list[-1]
            state.out_list = []
            if state.finished:
                if self.log_requests:
                    logger.info("Finish: obj=%s, out=%s", self._fmt_obj(obj), self._fmt_out(out))
                fr = out["meta_info"].get("finish_reason")
                if isinstance(fr, dict) and fr.get("type") == "abort" and fr.get("status_code") == 400:
                    raise ValueError(fr.get("message", "bad request"))
                yield out
                break
            state.event.clear()
            if obj.stream:
                yield out
            elif request is not None and await request.is_disconnected():
                self.abort_request(obj.rid)
                raise ValueError(f"Request is disconnected from the client side. Abort request rid={obj.rid}")

    async def _handle_batch_request(self, obj, request, created):
        bs = obj.batch_size
        gens, rids = [], []
        n = getattr(obj, "parallel_sample_num", 1)
        if n == 1:
            subs = [obj[i] for i in range(bs)]
            if getattr(self.server_args, "enable_tokenizer_batch_encode", False):
                toks = self._batch_tokenize(subs)          # one tokenizer call for the whole batch
            else:
                toks = [await self._tokenize_one_request(sub) for sub in subs]
            for sub, tok in zip(subs, toks):
                st = self._send_one_request(sub, tok, created)
                gens.append(self._wait_one_response(sub, st, request))
                rids.append(sub.rid)
        else:
            # Prefill each distinct prompt once with max_new_tokens = 0 so the n samples that
            # follow all hit the prefix cache instead of racing to compute the same prompt.
            objs = [obj[i] for i in range(bs)]
            toks = [await self._tokenize_one_request(o) for o in objs]
            for o, t in zip(objs, toks):
                warm_o = copy.copy(o)
                warm_o.rid = uuid.uuid4().hex
                warm_o.stream = False
                warm_t = copy.copy(t)
                warm_t.rid = warm_o.rid
                warm_t.sampling_params = copy.copy(t.sampling_params)
                warm_t.sampling_params.max_new_tokens = 0
                warm_t.stream = False
                st = self._send_one_request(warm_o, warm_t, created)
                async for _ in self._wait_one_response(warm_o, st, request):
                    pass
            for o, t in zip(objs, toks):
                for j in range(n):
                    so = copy.copy(o)
                    so.rid = uuid.uuid4().hex
                    stt = copy.copy(t)
                    stt.rid = so.rid
                    stt.sampling_params = copy.copy(t.sampling_params)
                    st = self._send_one_request(so, stt, created)
                    gens.append(self._wait_one_response(so, st, request))
                    rids.append(so.rid)
        if not obj.stream:
            outs = await asyncio.gather(*(g.__anext__() for g in gens))
            yield outs
        else:
            task_map = {asyncio.create_task(g.__anext__()): (i, g) for i, g in enumerate(gens)}
            while task_map:
                done, _ = await asyncio.wait(task_map.keys(), return_when=asyncio.FIRST_COMPLETED)
                for task in done:
                    i, g = task_map.pop(task)
                    try:
                        res = task.result()
                        res["index"] = i
                        yield res
                        task_map[asyncio.create_task(g.__anext__())] = (i, g)
                    except StopAsyncIteration:
                        pass

    # ------------------------------------------------------------------ control RPCs
    def abort_request(self, rid: str = "", abort_all: bool = False):
        if not abort_all and rid not in self.rid_to_state:
            return
        self.send_to_scheduler.send_pyobj(AbortReq(rid=rid, abort_all=abort_all))

    async def flush_cache(self) -> FlushCacheReqOutput:
        self.auto_create_handle_loop()
        return (await self.flush_cache_communicator(FlushCacheReqInput()))[0]

    async def pause_generation(self, obj: PauseGenerationReqInput):
        self.auto_create_handle_loop()
        async with self.is_pause_cond:
            self.is_pause = True
        self.send_to_scheduler.send_pyobj(obj)

    async def continue_generation(self, obj: ContinueGenerationReqInput):
        self.auto_create_handle_loop()
        async with self.is_pause_cond:
            self.is_pause = False
            self.send_to_scheduler.send_pyobj(obj)
            self.is_pause_cond.notify_all()

    # ------------------------------------------------------------------ LoRA (reference
    # `tokenizer_manager.py` load/unload_lora_adapter)
    async def load_lora_adapter(self, obj: LoadLoRAAdapterReqInput) -> LoRAUpdateOutput:
        self.auto_create_handle_loop()
        if self.lora_registry is None:
            return LoRAUpdateOutput(success=False, error_msg="LoRA is not enabled (--enable-lora)")
        if self.lora_update_lock is None:
            self.lora_update_lock = asyncio.Lock()
        from ..lora.lora_registry import LoRARef
        async with self.lora_update_lock:
            if self.lora_registry.get(obj.lora_name) is not None:
                return LoRAUpdateOutput(success=False, error_msg=f"LoRA adapter {obj.lora_name} is already loaded",
                                        loaded_adapters=self._loaded_loras())
            ref = LoRARef(lora_name=obj.lora_name, lora_path=obj.lora_path)
            obj.lora_id = ref.lora_id
            res = (await self.lora_communicator(obj))[0]
            if res.success:
                self.lora_registry.register(ref)
            res.loaded_adapters = self._loaded_loras()
            return res

    async def unload_lora_adapter(self, obj: UnloadLoRAAdapterReqInput) -> LoRAUpdateOutput:
        self.auto_create_handle_loop()
        if self.lora_registry is None:
            return LoRAUpdateOutput(success=False, error_msg="LoRA is not enabled (--enable-lora)")
        if self.lora_update_lock is None:
            self.lora_update_lock = asyncio.Lock()
        async with self.lora_update_lock:
            try:
                lora_id = self.lora_registry.unregister(obj.lora_name)
            except ValueError as e:
                return LoRAUpdateOutput(success=False, error_msg=str(e), loaded_adapters=self._loaded_loras())
            # new requests can no longer name the adapter; wait for the running ones
            await self.lora_registry.wait_for_unload(lora_id)
            obj.lora_id = lora_id
            res = (await self.lora_communicator(obj))[0]
            res.loaded_adapters = self._loaded_loras()
            return res

    def _loaded_loras(self) -> dict:
        return {n: r.lora_path for n, r in self.lora_registry.all().items()}

    async def get_internal_state(self) -> list[dict]:
        self.auto_create_handle_loop()
        return [r.internal_state for r in await self.get_internal_state_communicator(GetInternalStateReq())]

    async def set_internal_state(self, obj: SetInternalStateReq):
        self.auto_create_handle_loop()
        return await self.set_internal_state_communicator(obj)

    async def get_load(self):
        self.auto_create_handle_loop()
        return [dataclasses.asdict(r) for r in await self.get_load_communicator(GetLoadReqInput())]

    async def start_profile(self, output_dir=None, start_step=None, num_steps=None, profile_by_stage=False,
                            profile_stages=None, activities=None, profile_name=None, **kw):
        self.auto_create_handle_loop()
        req = ProfileReq(ProfileReqType.START_PROFILE, output_dir, start_step, num_steps,
                         profile_id=profile_name or str(time.time()), profile_by_stage=profile_by_stage,
                         profile_stages=profile_stages, activities=activities)
        res = (await self.profile_communicator(req))[0]
        if not res.success:
            raise RuntimeError(res.message)
        return res

    async def stop_profile(self):
        self.auto_create_handle_loop()
        res = (await self.profile_communicator(ProfileReq(ProfileReqType.STOP_PROFILE)))[0]
        if not res.success:
            raise RuntimeError(res.message)
        return res

    async def profile_status(self):
        self.auto_create_handle_loop()
        return (await self.profile_communicator(ProfileReq(ProfileReqType.STATUS)))[0]

    async def open_session(self, obj: OpenSessionReqInput):
        self.auto_create_handle_loop()
        if not obj.session_id:
            obj.session_id = uuid.uuid4().hex
        self.send_to_scheduler.send_pyobj(obj)
        return obj.session_id

    async def close_session(self, obj: CloseSessionReqInput):
        self.send_to_scheduler.send_pyobj(obj)

    def configure_logging(self, obj: ConfigureLoggingReq):
        if obj.log_requests is not None:
            self.log_requests = obj.log_requests
        if obj.log_requests_level is not None:
            self.log_requests_level = obj.log_requests_level
        if obj.log_level:
            logging.getLogger().setLevel(obj.log_level.upper())
            self.send_to_scheduler.send_pyobj(obj)

    async def score_request(self, query=None, items=None, label_token_ids=None, apply_softmax=False,
                            item_first=False, request=None) -> list[list[float]]:
        """Probabilities of `label_token_ids` as the next token after `query + item`
        (or `item + query`), one list per item."""
        if label_token_ids is None:
            raise ValueError("label_token_ids must be provided")
        if isinstance(query, str):
            prompts = [f"{it}{query}" if item_first else f"{query}{it}" for it in items]
            req = GenerateReqInput(text=prompts)
        else:
            prompts = [list(it) + list(query) if item_first else list(query) + list(it) for it in items]
            req = GenerateReqInput(input_ids=prompts)
        req.sampling_params = {"max_new_tokens": 1, "temperature": 0.0}
        req.return_logprob = True
        req.token_ids_logprob = list(label_token_ids)
        req.return_output_logprob_only = True
        req.stream = False
        results = await self.generate_request(req, request).__anext__()
        import math
        scores = []
        for r in results:
            lps = r["meta_info"].get("output_token_ids_logprobs", [[]])[0]
            m = {tid: lp for lp, tid, _ in lps}
            vals = [m.get(t, float("-inf")) for t in label_token_ids]
            if apply_softmax:
                mx = max(vals)
                ex = [math.exp(v - mx) if v != float("-inf") else 0.0 for v in vals]
                s = sum(ex) or 1.0
                scores.append([e / s for e in ex])
            else:
                scores.append([math.exp(v) if v != float("-inf") else 0.0 for v in vals])
        return scores

    # ------------------------------------------------------------------ receive loop
    def auto_create_handle_loop(self):
        if not self.to_create_loop:
            return
        self.to_create_loop = False
        self.loop = asyncio.get_running_loop()
        self.is_pause_cond = asyncio.Condition()
        if hasattr(self.recv_from_detokenizer, "q"):
            threading.Thread(target=self._queue_pump, daemon=True).start()
        else:
            self.loop.create_task(self.handle_loop())
        if self.crash_dump_folder:
            self.loop.create_task(self.sigterm_watchdog())

    def _queue_pump(self):
        while not self.gracefully_exit:
            try:
                obj = self.recv_from_detokenizer.recv_pyobj(timeout=0.1)
            except queue.Empty:
                continue
            self.loop.call_soon_threadsafe(self._dispatch_output, obj)

    async def handle_loop(self):
        while True:
            obj = await self.recv_from_detokenizer.recv_pyobj()
            self._dispatch_output(obj)

    def _dispatch_output(self, obj):
        self.last_receive_tstamp = time.time()
        if isinstance(obj, SchedulerFailure):
            self.fatal_error = obj.message or "the scheduler died"
            for st in list(self.rid_to_state.values()):
                st.event.set()
            return
        if isinstance(obj, (BatchStrOut, BatchEmbeddingOut)):
            self._handle_batch_output(obj)
            return
        fn = self._result_dispatch.get(type(obj))
        if fn is not None:
            fn(obj)

    def _handle_batch_output(self, recv):
        if getattr(recv, "cache_miss_count", None):
            if recv.cache_miss_count > self.cache_miss_count and os.environ.get("SGLANG_ENABLE_CACHE_MISS_CHECK"):
                raise RuntimeError(f"CUDA graphs were captured at serving time ({recv.cache_miss_count} captures)")
            self.cache_miss_count = recv.cache_miss_count
        for i, rid in enumerate(recv.rids):
            state = self.rid_to_state.get(rid)
            if state is None:
                continue
            fr = recv.finished_reasons[i]
            meta = {"id": rid, "finish_reason": fr, "prompt_tokens": recv.prompt_tokens[i]}
            if isinstance(recv, BatchStrOut):
                meta["completion_tokens"] = recv.completion_tokens[i]
                meta["cached_tokens"] = recv.cached_tokens[i]
                if getattr(state.obj, "return_logprob", False):
                    self.convert_logprob_style(meta, state, recv, i)
                if recv.output_hidden_states:
                    meta["hidden_states"] = recv.output_hidden_states[i]
                if recv.output_routed_experts:
                    meta["routed_experts"] = recv.output_routed_experts[i]
                if recv.spec_verify_ct:
                    meta["spec_verify_ct"] = recv.spec_verify_ct[i]
                if recv.dp_ranks:
                    meta["dp_rank"] = recv.dp_ranks[i]
                if recv.cache_miss_count is not None:
                    meta["cache_miss_count"] = recv.cache_miss_count
                if self.server_args.stream_output and fr is None:
                    state.text += recv.output_strs[i]
                    state.output_ids.extend(recv.output_ids[i])
                    out_ids = list(state.output_ids)
                    text = state.text
                elif self.server_args.stream_output:
                    text, out_ids = recv.output_strs[i], recv.output_ids[i]
                else:
                    text, out_ids = recv.output_strs[i], recv.output_ids[i]
                out = {"text": text, "output_ids": out_ids, "meta_info": meta}
            else:
                out = {"embedding": recv.embeddings[i], "meta_info": meta}
            if state.first_token_time == 0.0:
                state.first_token_time = time.time()
            state.finished = fr is not None
            if state.finished:
                state.finished_time = time.time()
                meta["e2e_latency"] = state.finished_time - state.created_time
                del self.rid_to_state[rid]
                if self.lora_registry is not None and getattr(state, "lora_id", None) is not None:
                    self.lora_registry.release(state.lora_id)
                if self.crash_dump_folder:
                    self.crash_dump_request_list.append((state.obj, out, state.created_time, time.time()))
                    if len(self.crash_dump_request_list) > 1000:
                        self.crash_dump_request_list.pop(0)
            state.out_list.append(out)
            state.event.set()
            if self.metrics_collector is not None and isinstance(recv, BatchStrOut):
                self.metrics_collector.observe(state, meta, state.finished)

    def convert_logprob_style(self, meta: dict, state: ReqState, recv: BatchStrOut, i: int):
        """Wire format -> API format: lists of `(logprob, token_id, token_text | None)`."""
        with_text = getattr(state.obj, "return_text_in_logprobs", False) and self.tokenizer is not None

        def conv(vals, idxs):
            if not vals:
                return []
            if with_text:
                texts = self.tokenizer.batch_decode([[t] for t in idxs])
                return list(zip(vals, idxs, texts))
            return [(v, t, None) for v, t in zip(vals, idxs)]

        def conv_top(vals, idxs):
            return [conv(v, x) if v else None for v, x in zip(vals or [], idxs or [])]

        if recv.input_token_logprobs_val and recv.input_token_logprobs_val[i]:
            state.input_token_logprobs = conv(recv.input_token_logprobs_val[i], recv.input_token_logprobs_idx[i])
            if recv.input_top_logprobs_val and recv.input_top_logprobs_val[i]:
                state.input_top_logprobs = conv_top(recv.input_top_logprobs_val[i], recv.input_top_logprobs_idx[i])
        if recv.output_token_logprobs_val:
            state.output_token_logprobs.extend(conv(recv.output_token_logprobs_val[i], recv.output_token_logprobs_idx[i]))
            if recv.output_top_logprobs_val and recv.output_top_logprobs_val[i]:
                state.output_top_logprobs.extend(conv_top(recv.output_top_logprobs_val[i], recv.output_top_logprobs_idx[i]))
            if recv.output_token_ids_logprobs_val and recv.output_token_ids_logprobs_val[i]:
                state.output_token_ids_logprobs.extend(
                    conv_top(recv.output_token_ids_logprobs_val[i], recv.output_token_ids_logprobs_idx[i]))
        meta["input_token_logprobs"] = state.input_token_logprobs
        meta["output_token_logprobs"] = state.output_token_logprobs
        if getattr(state.obj, "top_logprobs_num", 0):
            meta["input_top_logprobs"] = state.input_top_logprobs
            meta["output_top_logprobs"] = state.output_top_logprobs
        if getattr(state.obj, "token_ids_logprob", None):
            meta["input_token_ids_logprobs"] = state.input_token_ids_logprobs
            meta["output_token_ids_logprobs"] = state.output_token_ids_logprobs

    # ------------------------------------------------------------------ logging / forensics
    def _fmt_obj(self, obj) -> str:
        lvl = self.log_requests_level
        d = {k: v for k, v in dataclasses.asdict(obj).items() if v is not None} if dataclasses.is_dataclass(obj) else obj
        if lvl == 0:
            d = {k: v for k, v in d.items() if k in ("rid", "sampling_params", "stream")}
        elif lvl == 1:
            d = {k: v for k, v in d.items() if k not in ("text", "input_ids", "input_embeds", "image_data")}
        elif lvl == 2:
            d = {k: (str(v)[:2048] if k in ("text", "input_ids") else v) for k, v in d.items()}
        return str(d)

    def _fmt_out(self, out) -> str:
        lvl = self.log_requests_level
        if lvl == 0:
            return str({"meta_info": {k: v for k, v in out.get("meta_info", {}).items()
                                      if k in ("id", "finish_reason", "prompt_tokens", "completion_tokens")}})
        if lvl <= 2:
            o = dict(out)
            o["text"] = str(o.get("text", ""))[:2048]
            o.pop("output_ids", None)
            return str(o)
        return str(out)

    def dump_requests_before_crash(self):
        if not self.crash_dump_folder:
            return
        import pickle
        os.makedirs(self.crash_dump_folder, exist_ok=True)
        path = os.path.join(self.crash_dump_folder, f"crash_dump_{time.strftime('%Y%m%d_%H%M%S')}.pkl")
        unfinished = [(st.obj, {}, st.created_time, time.time()) for st in self.rid_to_state.values()]
        with open(path, "wb") as f:
            pickle.dump({"server_args": self.server_args.to_dict(),
                         "requests": self.crash_dump_request_list + unfinished}, f)
        logger.error("Dumped %d finished and %d unfinished requests to %s",
                     len(self.crash_dump_request_list), len(unfinished), path)

    async def sigterm_watchdog(self):
        while not self.gracefully_exit:
            await asyncio.sleep(5)
        # drain: wait for in-flight requests, then dump and exit
        while self.rid_to_state:
            await asyncio.sleep(1)
        self.dump_requests_before_crash()
