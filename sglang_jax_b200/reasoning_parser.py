"""Separates "thinking" text from the answer (reference `python/sgl_jax/srt/reasoning_parser.py`,
detector table :313-319).  Each model family has a start / end marker; some (DeepSeek-R1) start
in reasoning mode without emitting the start marker."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class StreamingParseResult:
    normal_text: str = ""
    reasoning_text: str = ""


class BaseReasoningFormatDetector:
    def __init__(self, think_start: str, think_end: str, force_reasoning: bool = False,
                 stream_reasoning: bool = True):
        self.think_start_token = think_start
        self.think_end_token = think_end
        self._in_reasoning = force_reasoning
        self.stream_reasoning = stream_reasoning
        self._buffer = ""
        self.stripped_think_start = False

    def detect_and_parse(self, text: str) -> StreamingParseResult:
        in_reasoning = self._in_reasoning or self.think_start_token in text
        if not in_reasoning:
            return StreamingParseResult(normal_text=text)
        processed = text.replace(self.think_start_token, "", 1).strip() if self.think_start_token in text else text
        if self.think_end_token not in processed:
            return StreamingParseResult(reasoning_text=processed)
        reasoning, normal = processed.split(self.think_end_token, 1)
        return StreamingParseResult(normal_text=normal.lstrip("\n"), reasoning_text=reasoning.rstrip())

    def parse_streaming_increment(self, new_text: str) -> StreamingParseResult:
        """Feed one streamed chunk.  A tail that could be the beginning of a marker is held back
        until the next chunk decides it."""
        cur = self._buffer + new_text
        keep = 0
        for tok in (self.think_start_token, self.think_end_token):
            for k in range(1, len(tok)):
                if cur.endswith(tok[:k]):
                    keep = max(keep, k)
        head, tail = (cur[: len(cur) - keep], cur[len(cur) - keep:]) if keep else (cur, "")
        res = self._process(head)
        self._buffer += tail
        return res

    def _process(self, cur: str) -> StreamingParseResult:
        self._buffer = ""
        if not self.stripped_think_start and self.think_start_token in cur:
            cur = cur.replace(self.think_start_token, "", 1)
            self.stripped_think_start = True
            self._in_reasoning = True
        if self._in_reasoning:
            if self.think_end_token in cur:
                reasoning, normal = cur.split(self.think_end_token, 1)
                self._in_reasoning = False
                return StreamingParseResult(normal_text=normal.lstrip("\n"), reasoning_text=reasoning)
            if self.stream_reasoning:
                return StreamingParseResult(reasoning_text=cur)
            self._buffer = cur
            return StreamingParseResult()
        return StreamingParseResult(normal_text=cur)


class DeepSeekR1Detector(BaseReasoningFormatDetector):
    def __init__(self, stream_reasoning=True, force_reasoning=True):
        super().__init__("<think>", "</think>", force_reasoning=True, stream_reasoning=stream_reasoning)


class Qwen3Detector(BaseReasoningFormatDetector):
    def __init__(self, stream_reasoning=True, force_reasoning=False):
        super().__init__("<think>", "</think>", force_reasoning=force_reasoning, stream_reasoning=stream_reasoning)


class KimiDetector(BaseReasoningFormatDetector):
    def __init__(self, stream_reasoning=True, force_reasoning=False):
        super().__init__("◁think▷", "◁/think▷", force_reasoning=force_reasoning, stream_reasoning=stream_reasoning)


class Gemma4Detector(BaseReasoningFormatDetector):
    def __init__(self, stream_reasoning=True, force_reasoning=False):
        super().__init__("<|channel>thought\n", "<channel|>", force_reasoning=force_reasoning,
                         stream_reasoning=stream_reasoning)


class ReasoningParser:
    DetectorMap = {
        "deepseek-r1": DeepSeekR1Detector, "deepseek-v3": Qwen3Detector, "qwen3": Qwen3Detector,
        "qwen3-thinking": DeepSeekR1Detector, "mimo": Qwen3Detector, "kimi": KimiDetector,
        "glm45": Qwen3Detector, "gemma4": Gemma4Detector, "step3": DeepSeekR1Detector,
    }

    def __init__(self, model_type: str | None = None, stream_reasoning: bool = True,
                 force_reasoning: bool | None = None):
        if not model_type:
            raise ValueError("Model type must be specified")
        cls = self.DetectorMap.get(model_type.lower())
        if cls is None:
            raise ValueError(f"Unsupported model type: {model_type}")
        kw = {"stream_reasoning": stream_reasoning}
        if force_reasoning is not None:
            kw["force_reasoning"] = force_reasoning
        self.detector = cls(**kw)

    def parse_non_stream(self, full_text: str) -> tuple[str, str]:
        r = self.detector.detect_and_parse(full_text)
        return r.reasoning_text, r.normal_text

    def parse_stream_chunk(self, chunk_text: str) -> tuple[str, str]:
        r = self.detector.parse_streaming_increment(chunk_text)
        return r.reasoning_text, r.normal_text
