"""In-process Python API.

Reference: `python/sgl_jax/srt/entrypoints/engine.py:71-736` — `Engine.generate` :150,
`async_generate` :201, `encode` :259, `rerank` :290, `shutdown` :303, pause/continue :353-367,
`abort_request` :370, profile :378, `get_server_info` :384, `score` :405,
`_launch_subprocesses` :555, `_launch_threads` :656.

Process model: the caller's process hosts the TokenizerManager; the Scheduler (with the
tensor-rank-0 model worker) and the DetokenizerManager run as subprocesses talking ZMQ, plus
one follower process per additional GPU.  With `enable_single_process=True` scheduler and
detokenizer are threads of the caller's process connected by queues (the mode tests, the
benchmark driver and RL-style embedding use).
"""

from __future__ import annotations

import asyncio
import atexit
import dataclasses
import logging
import multiprocessing as mp
import os
import queue
import signal
import threading
import time
from typing import Any, AsyncIterator, Iterator

from ..managers.io_struct import (CloseSessionReqInput, ConfigureLoggingReq, ContinueGenerationReqInput,
                                  EmbeddingReqInput, GenerateReqInput, OpenSessionReqInput,
                                  PauseGenerationReqInput, SetInternalStateReq)
from ..server_args import PortArgs, ServerArgs

logger = logging.getLogger(__name__)


class EngineBase:
    def generate(self, *a, **k):
        raise NotImplementedError

    def flush_cache(self):
        raise NotImplementedError

    def shutdown(self):
        raise NotImplementedError


class Engine(EngineBase):
    def __new__(cls, **kwargs):
        # dp_size > 1 runs as data-parallel attention under one scheduler (`managers/dp_scheduler.py`) when the
        # ranks are processes; in single-process mode, or with SGLB_DP_MODE=replicas, a set of independent
        # replicas behind a router stands in for the engine
        sa = kwargs.get("server_args")
        pd = sa.pd_disaggregation if sa is not None else kwargs.get("pd_disaggregation", "")
        mode = sa.disaggregation_mode if sa is not None else kwargs.get("disaggregation_mode", "null")
        if pd and mode in (None, "null") and not kwargs.get("_replica"):
            # `--pd-disaggregation`: prefill and decode engines of one node behind this one front door
            from ..disaggregation.local_pd import LocalPDEngine
            if sa is None:
                kwargs.setdefault("log_level", "error")
                sa = ServerArgs(**{k: v for k, v in kwargs.items() if k != "_replica"})
            return LocalPDEngine(sa)
        dp = sa.dp_size if sa is not None else int(kwargs.get("dp_size", 1) or 1)
        single = sa.enable_single_process if sa is not None else bool(kwargs.get("enable_single_process", False))
        replicas = single or os.environ.get("SGLB_DP_MODE", "attention") == "replicas"
        if dp > 1 and replicas and not kwargs.get("_replica"):
            from ..managers.data_parallel_controller import DataParallelEngine
            if sa is None:
                kwargs.setdefault("log_level", "error")
                sa = ServerArgs(**{k: v for k, v in kwargs.items() if k != "_replica"})
            return DataParallelEngine(sa)
        return super().__new__(cls)

    def __init__(self, **kwargs):
        kwargs.pop("_replica", None)
        if "server_args" in kwargs:
            server_args = kwargs["server_args"]
        else:
            if "log_level" not in kwargs:
                kwargs["log_level"] = "error"
            server_args = ServerArgs(**kwargs)
        self.server_args = server_args
        self._shutdown_done = False
        self.tokenizer_manager = None
        atexit.register(self.shutdown)
        self._threads: list[threading.Thread] = []
        self._procs: list[mp.Process] = []
        self._stop = threading.Event()
        self.scheduler = None
        self.loop = asyncio.new_event_loop()
        self._loop_thread = None
        if server_args.enable_engine_loop_run_forever_daemon:
            # the loop turns on a daemon thread of its own: the synchronous entry points hand it coroutines, so
            # `generate` can be called from several threads at once (reference `entrypoints/engine.py:133`)
            self._loop_thread = threading.Thread(target=self._loop_forever, daemon=True, name="engine-loop")
            self._loop_thread.start()
        if server_args.enable_single_process:
            self.tokenizer_manager, self.scheduler_info = _launch_threads(self, server_args)
        else:
            self.tokenizer_manager, self.scheduler_info = _launch_subprocesses(self, server_args)
        self.tokenizer_manager.max_req_input_len = self.scheduler_info.get("max_req_input_len")

    def _loop_forever(self):
        asyncio.set_event_loop(self.loop)
        self.loop.run_forever()

    def _run(self, coro):
        """Drive one coroutine of the tokenizer manager to completion from synchronous code."""
        if self._loop_thread is not None:
            return asyncio.run_coroutine_threadsafe(coro, self.loop).result()
        return self.loop.run_until_complete(coro)

    # ------------------------------------------------------------------ generation
    def _make_req(self, prompt, sampling_params, input_ids, return_logprob, logprob_start_len, top_logprobs_num,
                  token_ids_logprob, lora_path, stream, return_hidden_states, extra_key, **extra) -> GenerateReqInput:
        return GenerateReqInput(text=prompt, input_ids=input_ids, sampling_params=sampling_params,
                                return_logprob=return_logprob, logprob_start_len=logprob_start_len,
                                top_logprobs_num=top_logprobs_num, token_ids_logprob=token_ids_logprob,
                                lora_path=lora_path, stream=stream, return_hidden_states=return_hidden_states,
                                extra_key=extra_key, **extra)

    def generate(self, prompt: list[str] | str | None = None, sampling_params: list[dict] | dict | None = None,
                 input_ids: list[list[int]] | list[int] | None = None, return_logprob=False,
                 logprob_start_len=None, top_logprobs_num=None, token_ids_logprob=None, lora_path=None,
                 stream: bool = False, return_hidden_states: bool = False, extra_key=None, **extra
                 ) -> dict | list[dict] | Iterator[dict]:
        obj = self._make_req(prompt, sampling_params, input_ids, return_logprob, logprob_start_len,
                             top_logprobs_num, token_ids_logprob, lora_path, stream, return_hidden_states,
                             extra_key, **extra)
        gen = self.tokenizer_manager.generate_request(obj, None)
        if stream:
            def sync_iter():
                while True:
                    try:
                        yield self._run(gen.__anext__())
                    except StopAsyncIteration:
                        break
            return sync_iter()
        return self._run(gen.__anext__())

    async def async_generate(self, prompt=None, sampling_params=None, input_ids=None, return_logprob=False,
                             logprob_start_len=None, top_logprobs_num=None, token_ids_logprob=None, lora_path=None,
                             stream: bool = False, return_hidden_states: bool = False, extra_key=None, **extra
                             ) -> dict | AsyncIterator[dict]:
        obj = self._make_req(prompt, sampling_params, input_ids, return_logprob, logprob_start_len,
                             top_logprobs_num, token_ids_logprob, lora_path, stream, return_hidden_states,
                             extra_key, **extra)
        gen = self.tokenizer_manager.generate_request(obj, None)
        if stream:
            return gen
        return await gen.__anext__()

    def encode(self, prompt=None, input_ids=None, normalize: bool = True) -> dict | list[dict]:
        obj = EmbeddingReqInput(text=prompt, input_ids=input_ids, normalize=normalize)
        gen = self.tokenizer_manager.generate_request(obj, None)
        return self._run(gen.__anext__())

    def rerank(self, query: str, documents: list[str]) -> list[dict]:
        """Cross-encoder style scoring through the embedding path: one (query, document) pair per row."""
        outs = self.encode([f"{query}</s>{d}" for d in documents])
        scored = [{"index": i, "document": d, "score": float(o["embedding"][0])}
                  for i, (d, o) in enumerate(zip(documents, outs))]
        return sorted(scored, key=lambda x: -x["score"])

    def score(self, query=None, items=None, label_token_ids=None, apply_softmax=False, item_first=False):
        return self._run(self.tokenizer_manager.score_request(
            query, items, label_token_ids, apply_softmax, item_first))

    async def async_score(self, query=None, items=None, label_token_ids=None, apply_softmax=False, item_first=False):
        return await self.tokenizer_manager.score_request(query, items, label_token_ids, apply_softmax, item_first)

    # ------------------------------------------------------------------ control
    def flush_cache(self):
        return self._run(self.tokenizer_manager.flush_cache())

    def load_lora_adapter(self, lora_name: str, lora_path: str, pinned: bool = False):
        from ..managers.io_struct import LoadLoRAAdapterReqInput
        return self._run(self.tokenizer_manager.load_lora_adapter(
            LoadLoRAAdapterReqInput(lora_name=lora_name, lora_path=lora_path, pinned=pinned)))

    def unload_lora_adapter(self, lora_name: str):
        from ..managers.io_struct import UnloadLoRAAdapterReqInput
        return self._run(self.tokenizer_manager.unload_lora_adapter(
            UnloadLoRAAdapterReqInput(lora_name=lora_name)))

    def pause_generation(self, mode: str = "abort"):
        return self._run(self.tokenizer_manager.pause_generation(PauseGenerationReqInput(mode=mode)))

    def continue_generation(self):
        return self._run(self.tokenizer_manager.continue_generation(ContinueGenerationReqInput()))

    def abort_request(self, rid: str = "", abort_all: bool = False):
        self.tokenizer_manager.abort_request(rid, abort_all)

    def start_profile(self, **kw):
        return self._run(self.tokenizer_manager.start_profile(**kw))

    def stop_profile(self):
        return self._run(self.tokenizer_manager.stop_profile())

    def get_server_info(self) -> dict:
        internal = self._run(self.tokenizer_manager.get_internal_state())
        from .. import __version__
        return {**dataclasses.asdict(self.server_args), **self.scheduler_info, "internal_states": internal,
                "version": __version__}

    def get_load(self):
        return self._run(self.tokenizer_manager.get_load())

    def set_internal_state(self, **state):
        return self._run(self.tokenizer_manager.set_internal_state(
            SetInternalStateReq(state_data=state)))

    def open_session(self, session_id: str | None = None) -> str:
        return self._run(self.tokenizer_manager.open_session(
            OpenSessionReqInput(session_id=session_id or "")))

    def close_session(self, session_id: str):
        return self._run(self.tokenizer_manager.close_session(
            CloseSessionReqInput(session_id=session_id)))

    def release_memory_occupation(self):
        raise NotImplementedError("release_memory_occupation has no scheduler handler (as in the reference)")

    def resume_memory_occupation(self):
        raise NotImplementedError("resume_memory_occupation has no scheduler handler (as in the reference)")

    def get_default_sampling_params(self) -> dict:
        from ..sampling.sampling_params import SamplingParams
        return SamplingParams().convert_to_dict()

    def shutdown(self):
        if self._shutdown_done:
            return
        self._shutdown_done = True
        self._stop.set()
        if getattr(self, "tokenizer_manager", None) is not None:
            self.tokenizer_manager.gracefully_exit = True
        if self.scheduler is not None:
            try:
                self.scheduler.shutdown()
            except Exception:
                pass
        for t in self._threads:
            t.join(timeout=5)
        for p in self._procs:
            if p.is_alive():
                p.terminate()
        for p in self._procs:
            p.join(timeout=5)
            if p.is_alive():
                p.kill()
        # the tokenizer manager's receive loop is a task of this engine's event loop: cancel it and let the loop
        # run the cancellation, or the interpreter reports a destroyed pending task at exit
        loop = getattr(self, "loop", None)
        if getattr(self, "_loop_thread", None) is not None and loop is not None and loop.is_running():
            # run-forever mode: cancel the pending tasks on the loop's own thread, then stop it
            async def _cancel_all():
                tasks = [t for t in asyncio.all_tasks(loop) if t is not asyncio.current_task() and not t.done()]
                for t in tasks:
                    t.cancel()
                await asyncio.gather(*tasks, return_exceptions=True)
                await loop.shutdown_asyncgens()
            try:
                asyncio.run_coroutine_threadsafe(_cancel_all(), loop).result(timeout=5)
            except Exception:
                pass
            loop.call_soon_threadsafe(loop.stop)
            self._loop_thread.join(timeout=5)
            self._loop_thread = None
        elif loop is not None and not loop.is_closed() and not loop.is_running():
            try:
                tasks = [t for t in asyncio.all_tasks(loop) if not t.done()]
                for t in tasks:
                    t.cancel()
                if tasks:
                    loop.run_until_complete(asyncio.gather(*tasks, return_exceptions=True))
                loop.run_until_complete(loop.shutdown_asyncgens())
            except Exception:
                pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.shutdown()
        return False


# ------------------------------------------------------------------------------------ launchers
def _set_envs_and_config(server_args: ServerArgs):
    os.environ.setdefault("NCCL_CUMEM_ENABLE", "0")
    os.environ.setdefault("NCCL_NVLS_ENABLE", os.environ.get("NCCL_NVLS_ENABLE", "1"))
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "8")
    if threading.current_thread() is threading.main_thread():
        def on_child_quit(signum, frame):
            logger.error("A child process failed (SIGQUIT); shutting the engine down.")
            from ..utils.common import kill_process_tree
            kill_process_tree(os.getpid(), include_parent=True)

        try:
            signal.signal(signal.SIGQUIT, on_child_quit)
        except ValueError:
            pass
    try:
        mp.set_start_method("spawn", force=True)
    except RuntimeError:
        pass


def _launch_threads(engine: Engine, server_args: ServerArgs):
    """Scheduler + detokenizer as threads; queues instead of sockets."""
    from ..managers.communication import QueueReceiver, QueueSender
    from ..managers.detokenizer_manager import DetokenizerManager
    from ..managers.scheduler import Scheduler
    from ..managers.tokenizer_manager import TokenizerManager
    from ..parallel import state as ps
    from ..utils.common import configure_logger

    configure_logger(server_args)
    st = ps.get_state()
    own_state = None
    if server_args.device_indexes and server_args.tp_size == 1:
        # an engine pinned to one device of several: its scheduler thread gets a state of its own, so other engines
        # of this process (on other devices) are not disturbed
        own_state = ps.single_device_state(server_args.device, server_args.device_indexes[0])
    elif not st.initialized:
        if server_args.tp_size > 1:
            raise RuntimeError("enable_single_process with tp_size > 1 needs the ranks to be launched externally "
                               "(torchrun) and `parallel.state.init_distributed` called first")
        ps.init_distributed(0, 1, server_args.device)
    to_sched, to_detok, to_tok = queue.Queue(), queue.Queue(), queue.Queue()
    ready = threading.Event()
    info: dict[str, Any] = {}
    err: list[BaseException] = []

    def sched_main():
        try:
            import torch
            if own_state is not None:
                ps.bind_thread_state(own_state)
                engine.parallel_state = own_state
            if ps.get_state().device.type == "cuda":
                torch.cuda.set_device(ps.get_state().device)
            sched = Scheduler(server_args, None, recv_queue=to_sched, send_queue=_Router(to_detok, to_tok))
            engine.scheduler = sched
            info.update(max_total_num_tokens=sched.max_total_num_tokens, max_req_input_len=sched.max_req_input_len)
            ready.set()
            if sched.enable_overlap:
                sched.event_loop_overlap(engine._stop)
            else:
                sched.event_loop_normal(engine._stop)
        except BaseException as e:   # surface init failures to the caller, later ones to the requests
            from ..managers.io_struct import SchedulerFailure
            err.append(e)
            was_ready = ready.is_set()
            ready.set()
            logger.exception("scheduler thread died")
            if was_ready:
                to_tok.put(SchedulerFailure(f"{type(e).__name__}: {e}"))

    t = threading.Thread(target=sched_main, daemon=True, name="scheduler")
    t.start()
    engine._threads.append(t)
    ready.wait()
    if err:
        raise err[0]
    detok = DetokenizerManager(server_args, None, recv=QueueReceiver(to_detok), send=QueueSender(to_tok),
                               tokenizer=engine.scheduler.tokenizer)
    td = threading.Thread(target=detok.event_loop, args=(engine._stop,), daemon=True, name="detokenizer")
    td.start()
    engine._threads.append(td)
    tm = TokenizerManager(server_args, None, send_to_scheduler=QueueSender(to_sched),
                          recv_from_detokenizer=QueueReceiver(to_tok), tokenizer=engine.scheduler.tokenizer,
                          model_config=engine.scheduler.model_config)
    return tm, info


class _Router:
    """Scheduler output fan-out in single-process mode: token batches go to the detokenizer,
    control replies straight to the tokenizer manager."""

    def __init__(self, to_detok: queue.Queue, to_tok: queue.Queue):
        self.to_detok, self.to_tok = to_detok, to_tok

    def put(self, obj):
        from ..managers.io_struct import BatchEmbeddingOut, BatchTokenIDOut
        (self.to_detok if isinstance(obj, (BatchTokenIDOut, BatchEmbeddingOut)) else self.to_tok).put(obj)


def _launch_subprocesses(engine: Engine, server_args: ServerArgs):
    from ..managers.detokenizer_manager import run_detokenizer_process
    from ..managers.scheduler import run_scheduler_process
    from ..managers.tokenizer_manager import TokenizerManager
    from ..utils.common import configure_logger, get_free_port

    _set_envs_and_config(server_args)
    configure_logger(server_args)
    port_args = PortArgs.init_new(server_args)
    ranks_here = server_args.tp_size // server_args.nnodes
    first = server_args.node_rank * ranks_here
    if server_args.dist_init_addr:
        init_method = f"tcp://{server_args.dist_init_addr}"
    else:
        init_method = f"tcp://127.0.0.1:{get_free_port()}"
    readers = []
    for local in range(ranks_here):
        rank = first + local
        r, w = mp.Pipe(duplex=False)
        p = mp.Process(target=run_scheduler_process,
                       args=(server_args, port_args, w, rank, server_args.tp_size, init_method), daemon=False)
        p.start()
        engine._procs.append(p)
        readers.append(r)
    if server_args.node_rank >= 1:
        # follower node: no front-end; keep a health endpoint alive
        from ..utils.common import launch_dummy_health_check_server
        for r in readers:
            r.recv()
        launch_dummy_health_check_server(server_args.host, server_args.port)
        for p in engine._procs:
            p.join()
        return None, {}
    dp = mp.Process(target=run_detokenizer_process, args=(server_args, port_args), daemon=False)
    dp.start()
    engine._procs.append(dp)
    tm = TokenizerManager(server_args, port_args)
    info: dict[str, Any] = {}
    for i, r in enumerate(readers):
        deadline = time.time() + 3600
        while not r.poll(1.0):
            if not engine._procs[i].is_alive():
                raise RuntimeError(f"scheduler rank {first + i} died during initialisation "
                                   f"(exit code {engine._procs[i].exitcode})")
            if time.time() > deadline:
                raise TimeoutError("scheduler initialisation timed out")
        data = r.recv()
        if data.get("status") != "ready":
            raise RuntimeError("Initialization failed. Please see the error messages above.")
        if i == 0:
            info = {k: v for k, v in data.items() if k != "status"}
    return tm, info
