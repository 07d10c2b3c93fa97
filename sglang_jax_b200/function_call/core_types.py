"""Shared types of the tool-call parsers."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class ToolCallItem:
    tool_index: int
    name: str | None = None
    parameters: str = ""      # JSON text (possibly a fragment while streaming)


@dataclass
class StreamingParseResult:
    normal_text: str = ""
    calls: list[ToolCallItem] = field(default_factory=list)


@dataclass
class StructureInfo:
    begin: str
    end: str
    trigger: str
