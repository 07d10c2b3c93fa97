"""Front door of tool-call parsing (reference `python/sgl_jax/srt/function_call/function_call_parser.py`:
`FunctionCallParser` :22, detector map :31)."""

from __future__ import annotations

import json

from .core_types import ToolCallItem
from .detectors import Glm4MoeDetector, Glm47MoeDetector, MiMoDetector, Qwen3CoderDetector, Qwen25Detector
from .ebnf_composer import EBNFComposer


class FunctionCallParser:
    ToolCallParserEnum = {
        "qwen25": Qwen25Detector, "qwen": Qwen25Detector, "qwen3": Qwen25Detector,
        "qwen3_coder": Qwen3CoderDetector, "glm45": Glm4MoeDetector, "glm4_moe": Glm4MoeDetector,
        "glm47": Glm47MoeDetector, "glm47_moe": Glm47MoeDetector, "mimo": MiMoDetector,
    }

    def __init__(self, tools, tool_call_parser: str):
        cls = self.ToolCallParserEnum.get(tool_call_parser)
        if cls is None:
            raise ValueError(f"Unsupported tool_call_parser: {tool_call_parser}")
        self.detector = cls()
        self.tools = tools

    def has_tool_call(self, text: str) -> bool:
        return self.detector.has_tool_call(text)

    def parse_non_stream(self, full_text: str) -> tuple[str, list[ToolCallItem]]:
        r = self.detector.detect_and_parse(full_text, self.tools)
        return (r.normal_text, r.calls) if r.calls else (full_text, [])

    def parse_stream_chunk(self, chunk_text: str) -> tuple[str, list[ToolCallItem]]:
        r = self.detector.parse_streaming_increment(chunk_text, self.tools)
        return r.normal_text, r.calls

    def get_structure_tag(self) -> dict:
        get_info = self.detector.structure_info()
        structures, triggers = [], set()
        for t in self.tools:
            fn = t.function if hasattr(t, "function") else t["function"]
            name = fn.name if hasattr(fn, "name") else fn["name"]
            params = fn.parameters if hasattr(fn, "parameters") else fn.get("parameters")
            info = get_info(name)
            structures.append({"begin": info.begin, "schema": params or {}, "end": info.end})
            triggers.add(info.trigger)
        return {"type": "structural_tag", "structures": structures, "triggers": sorted(triggers)}

    def get_structure_constraint(self, tool_choice) -> tuple[str, str] | None:
        """(`kind`, `spec`) of the grammar that enforces `tool_choice`."""
        if tool_choice == "auto" and any(getattr(getattr(t, "function", None), "strict", False) for t in self.tools):
            return "structural_tag", json.dumps(self.get_structure_tag())
        if tool_choice == "required" or (not isinstance(tool_choice, str) and tool_choice is not None):
            fn_name = None
            if not isinstance(tool_choice, str):
                f = tool_choice.function if hasattr(tool_choice, "function") else tool_choice["function"]
                fn_name = f.name if hasattr(f, "name") else f["name"]
            d = self.detector
            return "ebnf", EBNFComposer.build_ebnf(self.tools, begin=d.bot_token, end=d.eot_token,
                                                   function_name=fn_name)
        return None
