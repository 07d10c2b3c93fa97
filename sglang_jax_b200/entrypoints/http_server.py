"""HTTP server: native, OpenAI-compatible and SageMaker-style routes.

Route set and semantics follow the reference's `python/sgl_jax/srt/entrypoints/http_server.py`
(app :134, `/health` :190 ... `/v1/rerank` :775, `launch` :785, warm-up :865)."""

from __future__ import annotations

import asyncio
import dataclasses
import json
import logging
import os
import threading
import time
from contextlib import asynccontextmanager
from typing import Any

import requests
from fastapi import FastAPI, Request
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import JSONResponse, Response, StreamingResponse

from ..function_call.function_call_parser import FunctionCallParser
from ..managers.io_struct import (CloseSessionReqInput, ConfigureLoggingReq, ContinueGenerationReqInput,
                                  EmbeddingReqInput, GenerateReqInput, LoadLoRAAdapterReqInput, OpenSessionReqInput,
                                  ParseFunctionCallReq, UnloadLoRAAdapterReqInput,
                                  PauseGenerationReqInput, ProfileReqInput, SeparateReasoningReqInput,
                                  SetInternalStateReq, StartTraceReqInput)
from ..managers.template_manager import TemplateManager
from ..reasoning_parser import ReasoningParser
from ..server_args import ServerArgs
from .openai.protocol import (ChatCompletionRequest, CompletionRequest, EmbeddingRequest, ModelCard, ModelList,
                              ScoringRequest, V1RerankReqInput)
from .openai.serving_chat import OpenAIServingChat
from .openai.serving_completions import OpenAIServingCompletion
from .openai.serving_embedding import OpenAIServingEmbedding, OpenAIServingRerank, OpenAIServingScore

logger = logging.getLogger(__name__)
HEALTH_CHECK_TIMEOUT = int(os.getenv("SGLANG_HEALTH_CHECK_TIMEOUT", 20))


@dataclasses.dataclass
class _GlobalState:
    tokenizer_manager: Any
    template_manager: TemplateManager
    scheduler_info: dict
    engine: Any = None


_global_state: _GlobalState | None = None


def set_global_state(state: _GlobalState):
    global _global_state
    _global_state = state


@asynccontextmanager
async def lifespan(app: FastAPI):
    tm = _global_state.tokenizer_manager
    app.state.completion = OpenAIServingCompletion(tm)
    app.state.chat = OpenAIServingChat(tm, _global_state.template_manager)
    app.state.embedding = OpenAIServingEmbedding(tm)
    app.state.rerank = OpenAIServingRerank(tm)
    app.state.score = OpenAIServingScore(tm)
    yield


app = FastAPI(lifespan=lifespan)
app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_credentials=True, allow_methods=["*"], allow_headers=["*"])


def _err(msg: str, code: int = 400):
    return JSONResponse({"error": {"message": msg}}, status_code=code)


# --------------------------------------------------------------------------- health / info
@app.get("/health")
async def health() -> Response:
    return Response(status_code=200)


@app.get("/ping")
async def ping() -> Response:
    return Response(status_code=200)


@app.get("/health_generate")
async def health_generate(request: Request) -> Response:
    """Generates one token; 503 if the scheduler does not answer in time."""
    tm = _global_state.tokenizer_manager
    rid = f"HEALTH_CHECK_{time.time()}"
    sp = {"max_new_tokens": 1, "temperature": 0.0}
    if tm.is_generation:
        gri = GenerateReqInput(rid=rid, input_ids=[0], sampling_params=sp)
    else:
        gri = EmbeddingReqInput(rid=rid, input_ids=[0])

    async def gen():
        async for _ in tm.generate_request(gri, request):
            break

    task = asyncio.create_task(gen())
    t0 = time.time()
    while time.time() < t0 + HEALTH_CHECK_TIMEOUT:
        await asyncio.sleep(0.05)
        if task.done() or tm.last_receive_tstamp > t0:
            task.cancel()
            tm.rid_to_state.pop(rid, None)
            return Response(status_code=200)
    task.cancel()
    tm.rid_to_state.pop(rid, None)
    logger.error("Health check failed. Server couldn't get a response from the scheduler in %ds", HEALTH_CHECK_TIMEOUT)
    return Response(status_code=503)


@app.get("/get_model_info")
async def get_model_info():
    tm = _global_state.tokenizer_manager
    return {"model_path": tm.model_path, "tokenizer_path": tm.server_args.tokenizer_path,
            "is_generation": tm.is_generation, "preferred_sampling_params": tm.server_args.preferred_sampling_params}


@app.get("/get_server_info")
async def get_server_info():
    from .. import __version__
    internal = await _global_state.tokenizer_manager.get_internal_state()
    return {**dataclasses.asdict(_global_state.tokenizer_manager.server_args), **_global_state.scheduler_info,
            "internal_states": internal, "version": __version__}


@app.get("/get_load")
async def get_load():
    return await _global_state.tokenizer_manager.get_load()


@app.api_route("/set_internal_state", methods=["POST", "PUT"])
async def set_internal_state(obj: dict, request: Request):
    res = await _global_state.tokenizer_manager.set_internal_state(SetInternalStateReq(state_data=obj.get("server_args", obj)))
    return {"updated": all(r.updated for r in res)}


# --------------------------------------------------------------------------- native generation
@app.api_route("/generate", methods=["POST", "PUT"])
async def generate_request(obj: dict, request: Request):
    try:
        gri = GenerateReqInput(**{k: v for k, v in obj.items() if k in GenerateReqInput.__dataclass_fields__})
    except TypeError as e:
        return _err(str(e))
    tm = _global_state.tokenizer_manager
    if gri.stream:
        async def stream_results():
            try:
                async for out in tm.generate_request(gri, request):
                    yield b"data: " + json.dumps(out, ensure_ascii=False).encode() + b"\n\n"
            except ValueError as e:
                yield b"data: " + json.dumps({"error": {"message": str(e)}}).encode() + b"\n\n"
            yield b"data: [DONE]\n\n"
        return StreamingResponse(stream_results(), media_type="text/event-stream")
    try:
        return await tm.generate_request(gri, request).__anext__()
    except ValueError as e:
        logger.error("[http_server] Error: %s", e)
        return _err(str(e))


@app.api_route("/generate_from_file", methods=["POST"])
async def generate_from_file_request(request: Request):
    """Body: raw bytes of a JSON file `{"input_ids"| "text": ..., "sampling_params": {...}}`."""
    try:
        obj = json.loads(await request.body())
        gri = GenerateReqInput(**{k: v for k, v in obj.items() if k in GenerateReqInput.__dataclass_fields__})
        return await _global_state.tokenizer_manager.generate_request(gri, request).__anext__()
    except ValueError as e:
        return _err(str(e))


@app.api_route("/encode", methods=["POST", "PUT"])
async def encode_request(obj: dict, request: Request):
    try:
        eri = EmbeddingReqInput(**{k: v for k, v in obj.items() if k in EmbeddingReqInput.__dataclass_fields__})
        return await _global_state.tokenizer_manager.generate_request(eri, request).__anext__()
    except ValueError as e:
        return _err(str(e))


@app.api_route("/classify", methods=["POST", "PUT"])
async def classify_request(obj: dict, request: Request):
    return await encode_request(obj, request)


# --------------------------------------------------------------------------- control
@app.api_route("/flush_cache", methods=["GET", "POST"])
async def flush_cache():
    ret = await _global_state.tokenizer_manager.flush_cache()
    return Response(content="Cache flushed.\nPlease check backend logs for more details. "
                            "(When there are running or waiting requests, the operation will not be performed.)\n",
                    status_code=200 if ret.success else 400)


@app.post("/load_lora_adapter")
async def load_lora_adapter(obj: LoadLoRAAdapterReqInput):
    res = await _global_state.tokenizer_manager.load_lora_adapter(obj)
    return JSONResponse(dataclasses.asdict(res), status_code=200 if res.success else 400)


@app.post("/unload_lora_adapter")
async def unload_lora_adapter(obj: UnloadLoRAAdapterReqInput):
    res = await _global_state.tokenizer_manager.unload_lora_adapter(obj)
    return JSONResponse(dataclasses.asdict(res), status_code=200 if res.success else 400)


@app.api_route("/start_profile", methods=["GET", "POST"])
async def start_profile_async(obj: ProfileReqInput | None = None):
    obj = obj or ProfileReqInput()
    try:
        await _global_state.tokenizer_manager.start_profile(
            output_dir=obj.output_dir, start_step=obj.start_step, num_steps=obj.num_steps,
            profile_by_stage=bool(obj.profile_by_stage), profile_stages=obj.profile_stages,
            activities=obj.activities, profile_name=obj.profile_name)
    except RuntimeError as e:
        return _err(str(e))
    return Response(content="Start profiling.\n", status_code=200)


@app.api_route("/stop_profile", methods=["GET", "POST"])
async def stop_profile_async():
    try:
        await _global_state.tokenizer_manager.stop_profile()
    except RuntimeError as e:
        return _err(str(e))
    return Response(content="Stop profiling. This will take some time.\n", status_code=200)


@app.api_route("/profile_status", methods=["GET"])
async def profile_status():
    res = await _global_state.tokenizer_manager.profile_status()
    return {"status": res.message}


@app.api_route("/start_trace", methods=["POST"])
async def start_trace(obj: StartTraceReqInput | None = None):
    """Precision tracer on: per-layer activation statistics are written as JSONL per request."""
    sa = _global_state.tokenizer_manager.server_args
    if not sa.enable_precision_tracer:
        return _err("Precision tracer is not enabled. Launch the server with --enable-precision-tracer.")
    obj = obj or StartTraceReqInput()
    state = {"enabled": True, "req_num": obj.req_num, "output_file": obj.output_file, "save_tensor": obj.save_tensor}
    await _global_state.tokenizer_manager.set_internal_state(SetInternalStateReq(state_data={"precision_tracer": state}))
    return {"status": "tracing", **state}


@app.api_route("/stop_trace", methods=["POST"])
async def stop_trace():
    await _global_state.tokenizer_manager.set_internal_state(
        SetInternalStateReq(state_data={"precision_tracer": {"enabled": False}}))
    return {"status": "stopped"}


@app.api_route("/trace_status", methods=["GET"])
async def trace_status():
    st = await _global_state.tokenizer_manager.get_internal_state()
    return st[0].get("precision_tracer", {"enabled": False})


@app.api_route("/release_memory_occupation", methods=["GET", "POST"])
async def release_memory_occupation():
    return _err("release_memory_occupation is not supported by the scheduler", 501)


@app.api_route("/resume_memory_occupation", methods=["GET", "POST"])
async def resume_memory_occupation():
    return _err("resume_memory_occupation is not supported by the scheduler", 501)


@app.api_route("/open_session", methods=["GET", "POST"])
async def open_session(obj: OpenSessionReqInput):
    sid = await _global_state.tokenizer_manager.open_session(obj)
    return sid


@app.api_route("/close_session", methods=["GET", "POST"])
async def close_session(obj: CloseSessionReqInput):
    await _global_state.tokenizer_manager.close_session(obj)
    return Response(status_code=200)


@app.api_route("/configure_logging", methods=["GET", "POST"])
async def configure_logging(obj: ConfigureLoggingReq):
    _global_state.tokenizer_manager.configure_logging(obj)
    return Response(status_code=200)


@app.post("/abort_request")
async def abort_request(obj: dict):
    _global_state.tokenizer_manager.abort_request(rid=obj.get("rid", ""), abort_all=bool(obj.get("abort_all", False)))
    return Response(status_code=200)


@app.post("/parse_function_call")
async def parse_function_call_request(obj: ParseFunctionCallReq):
    parser = FunctionCallParser(obj.tools or [], obj.tool_call_parser or _global_state.tokenizer_manager.server_args.tool_call_parser)
    normal, calls = parser.parse_non_stream(obj.text)
    return {"normal_text": normal, "calls": [dataclasses.asdict(c) for c in calls]}


@app.post("/separate_reasoning")
async def separate_reasoning_request(obj: SeparateReasoningReqInput):
    parser = ReasoningParser(obj.reasoning_parser or _global_state.tokenizer_manager.server_args.reasoning_parser)
    reasoning, text = parser.parse_non_stream(obj.text)
    return {"reasoning_text": reasoning, "text": text}


@app.post("/pause_generation")
async def pause_generation(obj: PauseGenerationReqInput | None = None):
    await _global_state.tokenizer_manager.pause_generation(obj or PauseGenerationReqInput())
    return {"message": "Generation paused successfully.", "status": "ok"}


@app.post("/continue_generation")
async def continue_generation(obj: ContinueGenerationReqInput | None = None):
    await _global_state.tokenizer_manager.continue_generation(obj or ContinueGenerationReqInput())
    return {"message": "Generation continued successfully.", "status": "ok"}


# --------------------------------------------------------------------------- OpenAI
@app.post("/v1/completions")
async def openai_v1_completions(request: CompletionRequest, raw_request: Request):
    return await raw_request.app.state.completion.handle_request(request, raw_request)


@app.post("/v1/chat/completions")
async def openai_v1_chat_completions(request: ChatCompletionRequest, raw_request: Request):
    return await raw_request.app.state.chat.handle_request(request, raw_request)


@app.post("/v1/embeddings")
async def openai_v1_embeddings(request: EmbeddingRequest, raw_request: Request):
    return await raw_request.app.state.embedding.handle_request(request, raw_request)


@app.get("/v1/models")
async def available_models():
    tm = _global_state.tokenizer_manager
    return ModelList(data=[ModelCard(id=tm.served_model_name, root=tm.served_model_name, max_model_len=tm.context_len)])


@app.get("/v1/models/{model:path}")
async def retrieve_model(model: str):
    tm = _global_state.tokenizer_manager
    if model != tm.served_model_name:
        return JSONResponse({"error": {"message": f"The model '{model}' does not exist", "type": "invalid_request_error",
                                       "param": "model", "code": "model_not_found"}}, status_code=404)
    return ModelCard(id=model, root=model, max_model_len=tm.context_len)


@app.post("/invocations")
async def sagemaker_chat_completions(request: ChatCompletionRequest, raw_request: Request):
    return await raw_request.app.state.chat.handle_request(request, raw_request)


@app.post("/v1/score")
async def v1_score_request(request: ScoringRequest, raw_request: Request):
    return await raw_request.app.state.score.handle_request(request, raw_request)


@app.post("/v1/rerank")
async def v1_rerank_request(request: V1RerankReqInput, raw_request: Request):
    return await raw_request.app.state.rerank.handle_request(request, raw_request)


# --------------------------------------------------------------------------- launch
def build_app_for_engine(engine) -> FastAPI:
    """Attach the FastAPI app to an existing `Engine` (tests use this with `TestClient`)."""
    tmpl = TemplateManager()
    tmpl.initialize_templates(engine.tokenizer_manager, engine.server_args.model_path)
    set_global_state(_GlobalState(engine.tokenizer_manager, tmpl, engine.scheduler_info, engine))
    return app


def launch(server_args: ServerArgs):
    """Start the engine processes, then serve HTTP until killed."""
    import uvicorn

    from ..utils.common import add_api_key_middleware, add_prometheus_middleware, set_prometheus_multiproc_dir
    from .engine import Engine
    if server_args.enable_metrics:
        set_prometheus_multiproc_dir()
    engine = Engine(server_args=server_args)
    if server_args.pd_disaggregation and server_args.disaggregation_mode in (None, "null"):
        # in-node PD launcher: the front door over the prefill and decode engines has its own small app
        from ..disaggregation.local_pd import build_pd_app
        try:
            uvicorn.run(build_pd_app(engine), host=server_args.host, port=server_args.port,
                        log_level=server_args.log_level_http or server_args.log_level, timeout_keep_alive=5)
        finally:
            engine.shutdown()
        return
    if engine.tokenizer_manager is None:
        return   # follower node
    build_app_for_engine(engine)
    if server_args.api_key:
        add_api_key_middleware(app, server_args.api_key)
    if server_args.enable_metrics:
        add_prometheus_middleware(app)
    threading.Thread(target=_wait_and_warmup, args=(server_args,), daemon=True).start()
    try:
        uvicorn.run(app, host=server_args.host, port=server_args.port,
                    log_level=server_args.log_level_http or server_args.log_level, timeout_keep_alive=5, loop="uvloop")
    finally:
        engine.shutdown()


def _execute_server_warmup(server_args: ServerArgs) -> bool:
    url = server_args.url()
    headers = {"Authorization": f"Bearer {server_args.api_key}"} if server_args.api_key else {}
    ok = False
    for _ in range(120):
        time.sleep(1)
        try:
            if requests.get(url + "/get_model_info", timeout=5, headers=headers).status_code == 200:
                ok = True
                break
        except requests.exceptions.RequestException:
            pass
    if not ok:
        logger.error("Initialization failed. warmup error: server did not come up")
        return False
    body = {"sampling_params": {"temperature": 0, "max_new_tokens": 8}}
    if server_args.skip_tokenizer_init:
        body["input_ids"] = [10, 11, 12]
    else:
        body["text"] = "The capital city of France is"
    try:
        r = requests.post(url + ("/generate" if not server_args.is_embedding else "/encode"), json=body,
                          headers=headers, timeout=600)
        return r.status_code == 200
    except Exception as e:
        logger.error("Initialization failed. warmup error: %s", e)
        return False


def _wait_and_warmup(server_args: ServerArgs):
    if not server_args.skip_server_warmup:
        if not _execute_server_warmup(server_args):
            return
    logger.info("The server is fired up and ready to roll!")
