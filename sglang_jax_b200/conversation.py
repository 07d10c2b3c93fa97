"""Plain-text conversation fallback used when a tokenizer ships no chat template (reference
`python/sgl_jax/srt/conversation.py`)."""

from __future__ import annotations

from typing import Any


def generate_chat_conv(messages: list[dict[str, Any]], tokenizer: Any = None, chat_template: str | None = None,
                       add_generation_prompt: bool = True) -> str:
    if tokenizer is not None and (chat_template or getattr(tokenizer, "chat_template", None)):
        return tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt,
                                             chat_template=chat_template)
    parts = []
    for m in messages:
        content = m.get("content", "")
        if isinstance(content, list):
            content = "".join(c.get("text", "") for c in content if isinstance(c, dict) and c.get("type") == "text")
        parts.append(f"{m.get('role', 'user')}: {content}")
    if add_generation_prompt:
        parts.append("assistant:")
    return "\n".join(parts)


class Conversation:
    def __init__(self, messages: list[dict[str, Any]] | None = None, system: str | None = None):
        self.messages: list[dict[str, Any]] = list(messages or [])
        if system:
            self.messages.insert(0, {"role": "system", "content": system})

    def add_message(self, role: str, content: str):
        self.messages.append({"role": role, "content": content})

    def get_prompt(self, tokenizer=None) -> str:
        return generate_chat_conv(self.messages, tokenizer)

    def clear(self):
        self.messages = []
