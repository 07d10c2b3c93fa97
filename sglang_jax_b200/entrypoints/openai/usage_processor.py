"""Token usage accounting for OpenAI responses (reference `entrypoints/openai/usage_processor.py`)."""

from __future__ import annotations

from .protocol import UsageInfo


class UsageProcessor:
    @staticmethod
    def calculate_response_usage(responses: list[dict], n_choices: int = 1, enable_cache_report: bool = False) -> UsageInfo:
        completion = sum(r["meta_info"].get("completion_tokens", 0) for r in responses)
        # with n > 1 every prompt appears n times in `responses`; count each prompt once
        prompt = sum(responses[i]["meta_info"].get("prompt_tokens", 0) for i in range(0, len(responses), max(n_choices, 1)))
        details = None
        if enable_cache_report:
            details = {"cached_tokens": sum(r["meta_info"].get("cached_tokens", 0) for r in responses)}
        return UsageInfo(prompt_tokens=prompt, completion_tokens=completion, total_tokens=prompt + completion,
                         prompt_tokens_details=details)

    @staticmethod
    def calculate_streaming_usage(prompt_tokens: dict[int, int], completion_tokens: dict[int, int],
                                  cached_tokens: dict[int, int], n_choices: int, enable_cache_report: bool = False) -> UsageInfo:
        prompt = sum(t for i, t in prompt_tokens.items() if i % max(n_choices, 1) == 0)
        completion = sum(completion_tokens.values())
        details = {"cached_tokens": sum(cached_tokens.values())} if enable_cache_report else None
        return UsageInfo(prompt_tokens=prompt, completion_tokens=completion, total_tokens=prompt + completion,
                         prompt_tokens_details=details)
