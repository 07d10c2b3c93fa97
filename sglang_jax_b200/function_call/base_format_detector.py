"""Base of the per-model tool-call detectors (reference
`python/sgl_jax/srt/function_call/base_format_detector.py`): one-shot parsing of a finished
message and incremental parsing of a stream, where a call's name is emitted as soon as it is
complete and its arguments are streamed as JSON text fragments."""

from __future__ import annotations

import json
import logging
from abc import ABC, abstractmethod

from .core_types import StreamingParseResult, StructureInfo, ToolCallItem

logger = logging.getLogger(__name__)


def _tool_names(tools) -> dict[str, int]:
    out = {}
    for i, t in enumerate(tools or []):
        fn = t.function if hasattr(t, "function") else t.get("function", {})
        name = fn.name if hasattr(fn, "name") else fn.get("name")
        if name:
            out[name] = i
    return out


def complete_partial_json(text: str) -> dict | list | None:
    """Best-effort parse of a JSON prefix: closes open strings / brackets."""
    try:
        return json.loads(text)
    except Exception:
        pass
    stack, in_str, esc = [], False, False
    for ch in text:
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
        elif ch == '"':
            in_str = True
        elif ch in "{[":
            stack.append("}" if ch == "{" else "]")
        elif ch in "}]" and stack:
            stack.pop()
    fixed = text + ('"' if in_str else "")
    fixed = fixed.rstrip()
    while fixed and fixed[-1] in ",:":
        fixed = fixed[:-1].rstrip()
        if fixed.endswith('"') and stack and stack[-1] == "}":
            # dangling key without value: drop it
            k = fixed.rfind('"', 0, len(fixed) - 1)
            fixed = fixed[:k].rstrip().rstrip(",")
    try:
        return json.loads(fixed + "".join(reversed(stack)))
    except Exception:
        return None


class BaseFormatDetector(ABC):
    bot_token = ""
    eot_token = ""
    tool_call_separator = ", "

    def __init__(self):
        self._buffer = ""
        self.current_tool_id = -1
        self.current_tool_name_sent = False
        self.streamed_args_for_tool: list[str] = []
        self.prev_tool_call_arr: list[dict] = []

    @abstractmethod
    def has_tool_call(self, text: str) -> bool: ...

    @abstractmethod
    def detect_and_parse(self, text: str, tools) -> StreamingParseResult: ...

    def parse_base_json(self, action, tools) -> list[ToolCallItem]:
        names = _tool_names(tools)
        out = []
        for act in action if isinstance(action, list) else [action]:
            name = act.get("name")
            if names and name not in names:
                logger.warning("Model attempted to call undefined function: %s", name)
                continue
            args = act.get("parameters", act.get("arguments", {}))
            out.append(ToolCallItem(tool_index=-1, name=name,
                                    parameters=args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)))
        return out

    def parse_streaming_increment(self, new_text: str, tools) -> StreamingParseResult:
        """Generic JSON-in-markers streaming: `bot_token {json} eot_token`."""
        self._buffer += new_text
        cur = self._buffer
        if self.bot_token and self.bot_token not in cur:
            # keep a tail that could start the marker
            keep = 0
            for k in range(1, len(self.bot_token)):
                if cur.endswith(self.bot_token[:k]):
                    keep = k
            self._buffer = cur[len(cur) - keep:] if keep else ""
            return StreamingParseResult(normal_text=cur[: len(cur) - keep] if keep else cur)
        start = cur.find(self.bot_token) if self.bot_token else 0
        normal = cur[:start]
        body = cur[start + len(self.bot_token):]
        end = body.find(self.eot_token) if self.eot_token else -1
        complete = end != -1
        json_text = body[:end] if complete else body
        res = StreamingParseResult(normal_text=normal)
        obj = complete_partial_json(json_text.strip())
        if self.current_tool_id == -1 or len(self.streamed_args_for_tool) <= self.current_tool_id:
            if self.current_tool_id == -1:
                self.current_tool_id = 0
            while len(self.streamed_args_for_tool) <= self.current_tool_id:
                self.streamed_args_for_tool.append("")
                self.prev_tool_call_arr.append({})
        if isinstance(obj, dict) and obj.get("name") and (not _tool_names(tools) or obj["name"] in _tool_names(tools)):
            if not self.current_tool_name_sent:
                if '"name"' in json_text and (complete or json_text.count('"') >= 4):
                    res.calls.append(ToolCallItem(self.current_tool_id, obj["name"], ""))
                    self.current_tool_name_sent = True
            if self.current_tool_name_sent:
                args = obj.get("arguments", obj.get("parameters"))
                if args is not None:
                    args_json = json.dumps(args, ensure_ascii=False)
                    if not complete:
                        # stream only the stable prefix: drop closing brackets the completer added
                        args_json = args_json.rstrip('}]"')
                    sent = self.streamed_args_for_tool[self.current_tool_id]
                    if args_json.startswith(sent) and len(args_json) > len(sent):
                        res.calls.append(ToolCallItem(self.current_tool_id, None, args_json[len(sent):]))
                        self.streamed_args_for_tool[self.current_tool_id] = args_json
                    self.prev_tool_call_arr[self.current_tool_id] = {"name": obj["name"], "arguments": args}
        if complete:
            self._buffer = body[end + len(self.eot_token):]
            self.current_tool_id += 1
            self.current_tool_name_sent = False
        else:
            self._buffer = cur[start:]
        return res

    def structure_info(self):
        return lambda name: StructureInfo(begin=f'{self.bot_token}{{"name":"{name}", "arguments":',
                                          end=f"}}{self.eot_token}", trigger=self.bot_token)

    def supports_structural_tag(self) -> bool:
        return True
