"""Helpers around Jinja chat templates (reference `python/sgl_jax/srt/jinja_template_utils.py`):
whether a template expects OpenAI-style content lists or plain strings, and normalising messages
accordingly."""

from __future__ import annotations

import re
from typing import Any

import jinja2


def detect_template_content_format(chat_template: str | None) -> str:
    """`"openai"` when the template iterates over `message.content` parts, else `"string"`."""
    if not chat_template:
        return "string"
    loops = re.findall(r"\{%-?\s*for\s+\w+\s+in\s+(\w+)(?:\.|\[['\"])content", chat_template)
    return "openai" if loops or re.search(r"content\s*\|\s*selectattr|item\.type|content\[\s*0\s*\]", chat_template) \
        else "string"


def process_content_for_template_format(msg: dict[str, Any], content_format: str, image_data: list | None = None,
                                        audio_data: list | None = None) -> dict[str, Any]:
    """Returns a copy of `msg` whose `content` matches what the template wants; media parts are
    collected into `image_data` / `audio_data` and replaced by typed placeholders."""
    content = msg.get("content")
    if not isinstance(content, list):
        return {k: v for k, v in msg.items() if v is not None}
    out = {k: v for k, v in msg.items() if k != "content" and v is not None}
    parts, text = [], []
    for c in content:
        if not isinstance(c, dict):
            continue
        t = c.get("type")
        if t == "text":
            parts.append({"type": "text", "text": c.get("text", "")})
            text.append(c.get("text", ""))
        elif t in ("image_url", "image"):
            if image_data is not None:
                image_data.append((c.get("image_url") or {}).get("url") if t == "image_url" else c.get("image"))
            parts.append({"type": "image"})
        elif t in ("audio_url", "input_audio", "audio"):
            if audio_data is not None:
                audio_data.append(c.get("audio_url") or c.get("input_audio") or c.get("audio"))
            parts.append({"type": "audio"})
    out["content"] = parts if content_format == "openai" else " ".join(text)
    return out


def render_template(template: str, **kwargs) -> str:
    env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True)
    env.globals["raise_exception"] = _raise
    return env.from_string(template).render(**kwargs)


def _raise(message: str):
    raise jinja2.exceptions.TemplateError(message)
