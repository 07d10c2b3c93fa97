"""Per-model tool-call formats (reference `python/sgl_jax/srt/function_call/{qwen25,qwen3_coder,
glm4_moe,glm47_moe,mimo}_detector.py`)."""

from __future__ import annotations

import json
import re

from .base_format_detector import BaseFormatDetector, _tool_names
from .core_types import StreamingParseResult, StructureInfo, ToolCallItem


class Qwen25Detector(BaseFormatDetector):
    """`<tool_call>\\n{"name": ..., "arguments": {...}}\\n</tool_call>`"""
    bot_token = "<tool_call>\n"
    eot_token = "\n</tool_call>"

    def has_tool_call(self, text: str) -> bool:
        return "<tool_call>" in text

    def detect_and_parse(self, text: str, tools) -> StreamingParseResult:
        idx = text.find("<tool_call>")
        if idx == -1:
            return StreamingParseResult(normal_text=text)
        normal = text[:idx].strip()
        calls = []
        for m in re.findall(r"<tool_call>\s*(.*?)\s*</tool_call>", text, re.DOTALL):
            try:
                calls.extend(self.parse_base_json(json.loads(m), tools))
            except json.JSONDecodeError:
                continue
        for i, c in enumerate(calls):
            c.tool_index = i
        return StreamingParseResult(normal_text=normal, calls=calls)


class MiMoDetector(Qwen25Detector):
    """MiMo uses the Qwen2.5 JSON-in-tags format."""


def _coerce(value: str, schema_type: str | None):
    v = value.strip()
    if schema_type in ("integer", "number", "boolean", "object", "array", "null"):
        try:
            return json.loads(v)
        except Exception:
            return v
    if schema_type == "string":
        return value.strip("\n")
    try:
        return json.loads(v)
    except Exception:
        return value.strip("\n")


def _param_types(tools, name) -> dict:
    for t in tools or []:
        fn = t.function if hasattr(t, "function") else t.get("function", {})
        fname = fn.name if hasattr(fn, "name") else fn.get("name")
        if fname == name:
            params = fn.parameters if hasattr(fn, "parameters") else fn.get("parameters")
            props = (params or {}).get("properties", {})
            return {k: v.get("type") for k, v in props.items() if isinstance(v, dict)}
    return {}


class _XmlStyleDetector(BaseFormatDetector):
    """Shared machinery of the XML-ish formats: whole calls are parsed once complete; the stream
    emits a call's name and its full arguments when the closing tag arrives."""
    call_re: re.Pattern

    def has_tool_call(self, text):
        return self.bot_token in text

    def _parse_call(self, body: str, tools) -> ToolCallItem | None:
        raise NotImplementedError

    def detect_and_parse(self, text, tools):
        idx = text.find(self.bot_token)
        if idx == -1:
            return StreamingParseResult(normal_text=text)
        calls = []
        for m in self.call_re.findall(text):
            c = self._parse_call(m, tools)
            if c is not None:
                c.tool_index = len(calls)
                calls.append(c)
        return StreamingParseResult(normal_text=text[:idx].strip(), calls=calls)

    def parse_streaming_increment(self, new_text, tools):
        self._buffer += new_text
        cur = self._buffer
        res = StreamingParseResult()
        while True:
            start = cur.find(self.bot_token)
            if start == -1:
                keep = 0
                for k in range(1, len(self.bot_token)):
                    if cur.endswith(self.bot_token[:k]):
                        keep = k
                res.normal_text += cur[: len(cur) - keep] if keep else cur
                cur = cur[len(cur) - keep:] if keep else ""
                break
            res.normal_text += cur[:start]
            end = cur.find(self.eot_token, start)
            if end == -1:
                cur = cur[start:]
                break
            body = cur[start + len(self.bot_token): end]
            c = self._parse_call(body, tools)
            if c is not None:
                self.current_tool_id += 1
                c.tool_index = self.current_tool_id
                res.calls.append(ToolCallItem(c.tool_index, c.name, ""))
                res.calls.append(ToolCallItem(c.tool_index, None, c.parameters))
                self.prev_tool_call_arr.append({"name": c.name, "arguments": json.loads(c.parameters)})
                self.streamed_args_for_tool.append(c.parameters)
            cur = cur[end + len(self.eot_token):]
        self._buffer = cur
        return res


class Qwen3CoderDetector(_XmlStyleDetector):
    """`<tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>`"""
    bot_token = "<tool_call>"
    eot_token = "</tool_call>"
    call_re = re.compile(r"<tool_call>(.*?)</tool_call>", re.DOTALL)

    def _parse_call(self, body, tools):
        m = re.search(r"<function=([^>\n]+)>(.*?)(?:</function>|$)", body, re.DOTALL)
        if not m:
            return None
        name = m.group(1).strip()
        if _tool_names(tools) and name not in _tool_names(tools):
            return None
        types = _param_types(tools, name)
        args = {}
        for k, v in re.findall(r"<parameter=([^>\n]+)>(.*?)</parameter>", m.group(2), re.DOTALL):
            args[k.strip()] = _coerce(v, types.get(k.strip()))
        return ToolCallItem(-1, name, json.dumps(args, ensure_ascii=False))

    def structure_info(self):
        return lambda name: StructureInfo(begin=f"<tool_call>\n<function={name}>\n", end="</function>\n</tool_call>",
                                          trigger="<tool_call>")


class Glm4MoeDetector(_XmlStyleDetector):
    """`<tool_call>NAME\\n<arg_key>K</arg_key>\\n<arg_value>V</arg_value>...</tool_call>`"""
    bot_token = "<tool_call>"
    eot_token = "</tool_call>"
    call_re = re.compile(r"<tool_call>(.*?)</tool_call>", re.DOTALL)

    def _parse_call(self, body, tools):
        m = re.match(r"\s*([^\n<]+)\s*(.*)", body, re.DOTALL)
        if not m:
            return None
        name = m.group(1).strip()
        if _tool_names(tools) and name not in _tool_names(tools):
            return None
        types = _param_types(tools, name)
        args = {}
        for k, v in re.findall(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", m.group(2), re.DOTALL):
            args[k.strip()] = _coerce(v, types.get(k.strip()))
        return ToolCallItem(-1, name, json.dumps(args, ensure_ascii=False))

    def structure_info(self):
        return lambda name: StructureInfo(begin=f"<tool_call>{name}\n", end="</tool_call>", trigger="<tool_call>")


class Glm47MoeDetector(Glm4MoeDetector):
    """GLM-4.7: same tags, the function name may be followed directly by the first `<arg_key>`."""

    def _parse_call(self, body, tools):
        m = re.match(r"\s*([^\n<]+?)\s*(<arg_key>.*)?$", body, re.DOTALL)
        if not m:
            return None
        return super()._parse_call(m.group(1) + "\n" + (m.group(2) or ""), tools)
