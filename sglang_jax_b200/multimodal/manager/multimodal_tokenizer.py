"""Front end of the multimodal server (reference `multimodal/manager/multimodal_tokenizer.py`):
turns API requests into tokenised stage-0 messages and resolves the futures when the pipeline
answers."""

from __future__ import annotations

import asyncio
import threading

from .io_struct import (GenerateMMReqInput, MMOutput, TokenizedGenerateMMReqInput)


class ByteTokenizer:
    """Fallback when a pipeline directory ships no tokenizer: UTF-8 bytes + 3 (0 pad, 1 eos, 2 unk)."""
    vocab_size = 259

    def encode(self, text: str) -> list[int]:
        return [b + 3 for b in text.encode("utf-8")] + [1]


class MultimodalTokenizer:
    def __init__(self, global_scheduler, tokenizer=None):
        self.gs = global_scheduler
        self.tokenizer = tokenizer or ByteTokenizer()
        self.pending: dict[str, tuple[asyncio.AbstractEventLoop, asyncio.Future]] = {}
        self._lock = threading.Lock()
        global_scheduler.on_output = self._on_output

    def _encode(self, text: str | None) -> list[int] | None:
        if text is None:
            return None
        t = self.tokenizer
        ids = t.encode(text)
        return list(ids.ids) if hasattr(ids, "ids") else list(ids)

    async def generate(self, obj: GenerateMMReqInput) -> MMOutput:
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        with self._lock:
            self.pending[obj.rid] = (loop, fut)
        self.gs.submit(TokenizedGenerateMMReqInput(
            rid=obj.rid, input_ids=self._encode(obj.prompt), negative_input_ids=self._encode(obj.negative_prompt),
            height=obj.height, width=obj.width, num_frames=obj.num_frames,
            num_inference_steps=obj.num_inference_steps, guidance_scale=obj.guidance_scale, seed=obj.seed,
            output_format=obj.output_format))
        return await fut

    def abort(self, rid: str):
        self.gs.abort(rid)

    def _on_output(self, out: MMOutput):
        with self._lock:
            ent = self.pending.pop(out.rid, None)
        if ent is not None:
            loop, fut = ent
            loop.call_soon_threadsafe(lambda: fut.done() or fut.set_result(out))
