"""`/v1/completions` (reference `entrypoints/openai/serving_completions.py`)."""

from __future__ import annotations

import time

from ...managers.io_struct import GenerateReqInput
from .protocol import (CompletionRequest, CompletionResponse, CompletionResponseChoice,
                       CompletionResponseStreamChoice, CompletionStreamResponse)
from .serving_base import OpenAIServingBase
from .usage_processor import UsageProcessor
from .utils import finish_reason_type, matched_stop, to_openai_style_logprobs


def build_sampling_params(request, stop=None, max_new_tokens=None) -> dict:
    sp = {
        "temperature": request.temperature, "max_new_tokens": max_new_tokens, "min_new_tokens": request.min_tokens,
        "stop": stop if stop is not None else request.stop, "stop_token_ids": request.stop_token_ids,
        "top_p": request.top_p, "top_k": request.top_k, "min_p": request.min_p,
        "presence_penalty": request.presence_penalty, "frequency_penalty": request.frequency_penalty,
        "repetition_penalty": request.repetition_penalty, "regex": request.regex, "json_schema": request.json_schema,
        "ebnf": request.ebnf, "n": request.n, "no_stop_trim": request.no_stop_trim, "ignore_eos": request.ignore_eos,
        "skip_special_tokens": request.skip_special_tokens, "logit_bias": request.logit_bias,
        "sampling_seed": request.sampling_seed if request.sampling_seed is not None else request.seed,
    }
    rf = getattr(request, "response_format", None)
    if rf is not None:
        import json
        if rf.type == "json_schema" and rf.json_schema is not None:
            sp["json_schema"] = json.dumps(rf.json_schema.schema_)
        elif rf.type == "json_object":
            sp["json_schema"] = '{"type": "object"}'
        elif rf.type == "structural_tag":
            sp["structural_tag"] = json.dumps(rf.model_dump(by_alias=True))
    return sp


class OpenAIServingCompletion(OpenAIServingBase):
    def _validate_request(self, request: CompletionRequest):
        if request.prompt is None or (isinstance(request.prompt, (list, str)) and len(request.prompt) == 0):
            return "Prompt cannot be empty"
        if request.n < 1:
            return "n must be at least 1"
        return None

    def _convert_to_internal_request(self, request: CompletionRequest):
        prompt = request.prompt
        kw = {}
        if isinstance(prompt, str) or (isinstance(prompt, list) and prompt and isinstance(prompt[0], str)):
            kw["text"] = prompt
        else:
            kw["input_ids"] = prompt
        logprob_start_len = -1
        if request.echo and request.logprobs is not None:
            logprob_start_len = 0
        adapted = GenerateReqInput(
            **kw, sampling_params=build_sampling_params(request, max_new_tokens=request.max_tokens),
            return_logprob=request.logprobs is not None, top_logprobs_num=request.logprobs or 0,
            logprob_start_len=logprob_start_len, return_text_in_logprobs=True, stream=request.stream,
            lora_path=request.lora_path, rid=request.rid, extra_key=request.extra_key,
            return_hidden_states=request.return_hidden_states, return_routed_experts=request.return_routed_experts,
            bootstrap_host=request.bootstrap_host, bootstrap_port=request.bootstrap_port,
            bootstrap_room=request.bootstrap_room)
        return adapted, request

    def _echo_text(self, request, index: int) -> str:
        p = request.prompt
        tok = self.tokenizer_manager.tokenizer
        if isinstance(p, str):
            return p
        if isinstance(p, list) and p and isinstance(p[0], str):
            return p[index // request.n]
        if isinstance(p, list) and p and isinstance(p[0], int):
            return tok.decode(p, skip_special_tokens=True) if tok else ""
        return tok.decode(p[index // request.n], skip_special_tokens=True) if tok else ""

    async def _handle_non_streaming_request(self, adapted, request, raw_request):
        ret = await self.tokenizer_manager.generate_request(adapted, raw_request).__anext__()
        if not isinstance(ret, list):
            ret = [ret]
        choices = []
        for idx, item in enumerate(ret):
            text = item["text"]
            if request.echo:
                text = self._echo_text(request, idx) + text
            lp = None
            if request.logprobs is not None:
                mi = item["meta_info"]
                lp = to_openai_style_logprobs(
                    input_token_logprobs=mi.get("input_token_logprobs") if request.echo else None,
                    input_top_logprobs=mi.get("input_top_logprobs") if request.echo else None,
                    output_token_logprobs=mi.get("output_token_logprobs"),
                    output_top_logprobs=mi.get("output_top_logprobs"))
            fr = item["meta_info"]["finish_reason"]
            choices.append(CompletionResponseChoice(index=idx, text=text, logprobs=lp,
                                                    finish_reason=finish_reason_type(fr), matched_stop=matched_stop(fr),
                                                    hidden_states=item["meta_info"].get("hidden_states")))
        usage = UsageProcessor.calculate_response_usage(ret, request.n, self.tokenizer_manager.server_args.enable_cache_report)
        return CompletionResponse(id=ret[0]["meta_info"]["id"], model=request.model, created=int(time.time()),
                                  choices=choices, usage=usage)

    async def _generate_stream(self, adapted, request, raw_request):
        created = int(time.time())
        stream_buffers, n_prev_tokens = {}, {}
        prompt_tokens, completion_tokens, cached_tokens = {}, {}, {}
        try:
            async for content in self.tokenizer_manager.generate_request(adapted, raw_request):
                index = content.get("index", 0)
                text = content["text"]
                mi = content["meta_info"]
                prompt_tokens[index] = mi["prompt_tokens"]
                completion_tokens[index] = mi["completion_tokens"]
                cached_tokens[index] = mi.get("cached_tokens", 0)
                buf = stream_buffers.get(index, "")
                if not buf and request.echo:
                    text = self._echo_text(request, index) + text
                lp = None
                if request.logprobs is not None:
                    n_prev = n_prev_tokens.get(index, 0)
                    lp = to_openai_style_logprobs(
                        output_token_logprobs=mi.get("output_token_logprobs", [])[n_prev:],
                        output_top_logprobs=(mi.get("output_top_logprobs") or [])[n_prev:])
                    n_prev_tokens[index] = len(mi.get("output_token_logprobs", []))
                delta = text[len(buf):]
                stream_buffers[index] = buf + delta
                fr = mi["finish_reason"]
                chunk = CompletionStreamResponse(
                    id=mi["id"], created=created, model=request.model,
                    choices=[CompletionResponseStreamChoice(index=index, text=delta, logprobs=lp,
                                                            finish_reason=finish_reason_type(fr),
                                                            matched_stop=matched_stop(fr))])
                yield f"data: {chunk.model_dump_json()}\n\n"
            if request.stream_options and request.stream_options.include_usage:
                usage = UsageProcessor.calculate_streaming_usage(prompt_tokens, completion_tokens, cached_tokens,
                                                                 request.n, self.tokenizer_manager.server_args.enable_cache_report)
                final = CompletionStreamResponse(id=mi["id"], created=created, model=request.model, choices=[], usage=usage)
                yield f"data: {final.model_dump_json(exclude_none=True)}\n\n"
        except Exception as e:
            yield f"data: {self.create_streaming_error_response(str(e))}\n\n"
        yield "data: [DONE]\n\n"
