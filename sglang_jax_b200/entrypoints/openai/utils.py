"""Helpers shared by the OpenAI handlers (reference `entrypoints/openai/utils.py`)."""

from __future__ import annotations

from .protocol import ChatCompletionTokenLogprob, ChoiceLogprobs, LogProbs, TopLogprob


def to_openai_style_logprobs(input_token_logprobs=None, output_token_logprobs=None, input_top_logprobs=None,
                             output_top_logprobs=None) -> LogProbs:
    ret = LogProbs()

    def add_tokens(lps):
        for lp, _tid, text in lps:
            ret.tokens.append(text if text is not None else str(_tid))
            ret.token_logprobs.append(lp)
            ret.text_offset.append(-1)

    def add_top(tops):
        for t in tops:
            ret.top_logprobs.append({(x[2] if x[2] is not None else str(x[1])): x[0] for x in t} if t else None)

    if input_token_logprobs:
        add_tokens(input_token_logprobs)
    if input_top_logprobs:
        add_top(input_top_logprobs)
    if output_token_logprobs:
        add_tokens(output_token_logprobs)
    if output_top_logprobs:
        add_top(output_top_logprobs)
    return ret


def to_chat_logprobs(output_token_logprobs, output_top_logprobs) -> ChoiceLogprobs:
    content = []
    for i, (lp, tid, text) in enumerate(output_token_logprobs or []):
        tok = text if text is not None else str(tid)
        tops = []
        if output_top_logprobs and i < len(output_top_logprobs) and output_top_logprobs[i]:
            for tlp, ttid, ttext in output_top_logprobs[i]:
                tt = ttext if ttext is not None else str(ttid)
                tops.append(TopLogprob(token=tt, bytes=list(tt.encode()), logprob=tlp))
        content.append(ChatCompletionTokenLogprob(token=tok, bytes=list(tok.encode()), logprob=lp, top_logprobs=tops))
    return ChoiceLogprobs(content=content)


def finish_reason_type(fr: dict | None) -> str | None:
    return fr["type"] if fr else None


def matched_stop(fr: dict | None):
    return fr.get("matched") if fr else None
