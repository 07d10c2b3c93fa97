"""HTTP front end of the multimodal server (reference `multimodal/entrypoint/http_server.py`:
`/api/v1/images/generation` :55, `/api/v1/videos/generation` :187, `/v1/audio/speech` :204,
`/v1/audio/transcriptions` :280, `/v1/chat/completions` :300, `/abort_request` :350)."""

from __future__ import annotations

import asyncio
import base64
import logging
import uuid

import numpy as np
from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, Response

from ..configs.stage_config import resolve
from ..manager.global_scheduler import GlobalScheduler
from ..manager.io_struct import (GenerateMMReqInput, MMOutput, TokenizedGenerateAudioReqInput,
                                 TokenizedGenerateOmniReqInput)
from ..manager.multimodal_detokenizer import MultimodalDetokenizer
from ..manager.multimodal_tokenizer import MultimodalTokenizer

logger = logging.getLogger(__name__)


class MultimodalServer:
    def __init__(self, pipeline: str, model_dir: str | None = None, config_overrides: dict | None = None,
                 tokenizer=None):
        self.pipeline = resolve(pipeline)
        self.gs = GlobalScheduler(self.pipeline, model_dir, config_overrides=config_overrides).start()
        self.tok = MultimodalTokenizer(self.gs, tokenizer)
        self.detok = MultimodalDetokenizer()
        self.kinds = {s.scheduler for s in self.pipeline.stages}
        from ..manager.multimodal_tokenizer import MediaPreprocessor
        self.media = MediaPreprocessor(model_dir, (config_overrides or {}).get("media"))

    async def _await(self, rid: str, submit) -> MMOutput:
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        with self.tok._lock:
            self.tok.pending[rid] = (loop, fut)
        submit()
        return await fut

    def shutdown(self):
        self.gs.shutdown()


def build_app(server: MultimodalServer) -> FastAPI:
    app = FastAPI(title="sglang multimodal")
    app.state.server = server

    def fail(out: MMOutput):
        code = 499 if out.error == "aborted" else 500
        return JSONResponse({"error": {"message": out.error, "rid": out.rid}}, status_code=code)

    def need(kind: str):
        if kind not in server.kinds:
            return JSONResponse({"error": {"message": f"the loaded pipeline ({server.pipeline.model_arch}) has no "
                                                      f"{kind} stage"}}, status_code=400)
        return None

    @app.get("/health")
    async def health():
        return {"status": "ok", "model_arch": server.pipeline.model_arch,
                "stages": [{"id": s.config.stage_id, "scheduler": s.config.scheduler, "devices": s.devices,
                            "processed": s.processed} for s in server.gs.stages]}

    async def _generate_visual(body: dict, video: bool):
        if (r := need("diffusion")) is not None:
            return r
        size = str(body.get("size", "64x64")).lower().split("x")
        obj = GenerateMMReqInput(
            prompt=body.get("prompt", ""), negative_prompt=body.get("negative_prompt"),
            width=int(body.get("width", size[0])), height=int(body.get("height", size[-1])),
            num_frames=int(body.get("num_frames", 9 if video else 1)),
            num_inference_steps=int(body.get("num_inference_steps", 8)),
            guidance_scale=float(body.get("guidance_scale", 1.0)), seed=int(body.get("seed", 0)),
            output_format=body.get("response_format", "b64_png"), rid=body.get("rid") or uuid.uuid4().hex)
        out = await server.tok.generate(obj)
        if out.error:
            return fail(out)
        payload = server.detok.image_payload(out.result["pixels"], obj.output_format)
        return {"id": out.rid, "data": payload, "meta": out.meta}

    @app.post("/api/v1/images/generation")
    async def images(request: Request):
        return await _generate_visual(await request.json(), False)

    @app.post("/api/v1/videos/generation")
    async def videos(request: Request):
        return await _generate_visual(await request.json(), True)

    @app.post("/v1/audio/speech")
    async def speech(request: Request):
        if (r := need("audio_decoder")) is not None:
            return r
        b = await request.json()
        rid = b.get("rid") or uuid.uuid4().hex
        ids = server.tok._encode(b.get("input", ""))
        sp = {"max_new_tokens": int(b.get("max_new_tokens", 32)), "temperature": float(b.get("temperature", 0.0))}
        out = await server._await(rid, lambda: server.gs.submit(
            TokenizedGenerateAudioReqInput(rid, ids, None, "tts", sp)))
        if out.error:
            return fail(out)
        wav = server.detok.audio_payload(out.result["waveform"].numpy())
        return Response(content=wav, media_type="audio/wav")

    @app.post("/v1/audio/transcriptions")
    async def transcriptions(request: Request):
        if (r := need("audio_encoder")) is not None:
            return r
        b = await request.json()
        rid = b.get("rid") or uuid.uuid4().hex
        wave = np.frombuffer(base64.b64decode(b["audio_b64"]), dtype="<f4") if "audio_b64" in b else np.asarray(b["audio"], np.float32)
        sp = {"max_new_tokens": int(b.get("max_new_tokens", 32)), "temperature": 0.0}
        out = await server._await(rid, lambda: server.gs.submit(
            TokenizedGenerateAudioReqInput(rid, server.tok._encode(b.get("prompt", "")), wave, "asr", sp)))
        if out.error:
            return fail(out)
        ids = out.result["output_ids"]
        text = bytes(t - 3 for t in ids if 3 <= t < 259).decode("utf-8", errors="replace")
        return {"text": text, "output_ids": ids}

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        if "auto_regressive" not in server.kinds and (r := need("llm")) is not None:
            return r
        b = await request.json()
        rid = b.get("rid") or uuid.uuid4().hex
        sp = {"max_new_tokens": int(b.get("max_tokens", 16)), "temperature": float(b.get("temperature", 0.0))}
        if b.get("images") or b.get("audios"):
            # raw media (base64 / data-URI images, PCM sample lists): preprocess here and expand the
            # single placeholder tokens of the prompt
            try:
                audios = [np.frombuffer(base64.b64decode(a), dtype="<f4") if isinstance(a, str) else a
                          for a in (b.get("audios") or [])]
                m = server.media(list(b["input_ids"]), b.get("images"), audios)
            except (ValueError, KeyError) as e:
                return JSONResponse({"error": {"message": str(e), "code": 400}}, status_code=400)
            req = TokenizedGenerateOmniReqInput(rid, m["input_ids"], m.get("pixel_values"), m.get("image_grid_thw"),
                                                m.get("audio_features"), sp, m.get("audio_feature_lens"))
        else:
            req = TokenizedGenerateOmniReqInput(
                rid, list(b["input_ids"]),
                np.asarray(b["pixel_values"], np.float32) if b.get("pixel_values") is not None else None,
                np.asarray(b["image_grid_thw"]) if b.get("image_grid_thw") is not None else None,
                np.asarray(b["audio_features"], np.float32) if b.get("audio_features") is not None else None, sp)
        out = await server._await(rid, lambda: server.gs.submit(req))
        if out.error:
            return fail(out)
        return {"id": out.rid, "object": "chat.completion",
                "choices": [{"index": 0, "message": {"role": "assistant", "content": None,
                                                     "output_ids": out.result["output_ids"]}, "finish_reason": "length"}]}

    @app.post("/abort_request")
    async def abort(request: Request):
        b = await request.json()
        return {"aborted": bool(server.gs.abort(b.get("rid", "")))}

    return app


def launch(pipeline: str, model_dir: str | None = None, host: str = "0.0.0.0", port: int = 30010, **kw):
    import uvicorn
    uvicorn.run(build_app(MultimodalServer(pipeline, model_dir, **kw)), host=host, port=port, log_level="info")
