"""Chat / completion template selection (reference `python/sgl_jax/srt/managers/template_manager.py`,
`conversation.py`, `jinja_template_utils.py`): the tokenizer's own Jinja chat template by default,
`--chat-template` style overrides from a file, and a minimal built-in ChatML fallback."""

from __future__ import annotations

import json
import logging
import os

logger = logging.getLogger(__name__)

CHATML = ("{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
          "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}")


class TemplateManager:
    def __init__(self):
        self.chat_template_name: str | None = None
        self.jinja_template: str | None = None
        self.jinja_template_content_format = "string"

    def initialize_templates(self, tokenizer_manager, model_path: str, chat_template: str | None = None,
                             completion_template: str | None = None):
        tok = tokenizer_manager.tokenizer
        if chat_template:
            if os.path.isfile(chat_template):
                with open(chat_template) as f:
                    text = f.read()
                if chat_template.endswith(".json"):
                    text = json.loads(text).get("chat_template", text)
                self.jinja_template = text
            elif chat_template == "chatml":
                self.jinja_template = CHATML
            else:
                raise ValueError(f"unknown chat template {chat_template}")
        elif tok is not None and getattr(tok, "chat_template", None):
            self.jinja_template = None    # tokenizer's own
        else:
            self.jinja_template = CHATML
        self.jinja_template_content_format = detect_content_format(
            self.jinja_template or getattr(tok, "chat_template", "") or "")

    def apply(self, tokenizer, messages: list[dict], tools=None, add_generation_prompt=True, **kwargs) -> list[int] | str:
        if tokenizer is None:
            raise ValueError("chat completions need a tokenizer (do not use --skip-tokenizer-init)")
        kw = dict(tokenize=True, add_generation_prompt=add_generation_prompt, **kwargs)
        if tools:
            kw["tools"] = tools
        if self.jinja_template is not None:
            kw["chat_template"] = self.jinja_template
        out = tokenizer.apply_chat_template(messages, **kw)
        if isinstance(out, dict):
            out = out["input_ids"]
        return out


def detect_content_format(template: str) -> str:
    """"openai" when the template iterates over content parts, else "string"."""
    if not template:
        return "string"
    return "openai" if ("content" in template and ("for" in template and "['type']" in template or
                                                    ".type" in template and "for" in template)) else "string"


def flatten_content(content) -> str:
    if content is None or isinstance(content, str):
        return content or ""
    parts = []
    for p in content:
        t = p.get("type") if isinstance(p, dict) else getattr(p, "type", None)
        if t == "text":
            parts.append(p["text"] if isinstance(p, dict) else p.text)
    return "\n".join(parts)
