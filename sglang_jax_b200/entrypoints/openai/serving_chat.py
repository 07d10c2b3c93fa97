"""`/v1/chat/completions` (reference `entrypoints/openai/serving_chat.py`): chat template,
tools -> grammar constraint, reasoning separation and tool-call parsing, both streaming and not."""

from __future__ import annotations

import json
import time
import uuid

from ...function_call.function_call_parser import FunctionCallParser
from ...managers.io_struct import GenerateReqInput
from ...managers.template_manager import flatten_content
from ...reasoning_parser import ReasoningParser
from .protocol import (ChatCompletionRequest, ChatCompletionResponse, ChatCompletionResponseChoice,
                       ChatCompletionResponseStreamChoice, ChatCompletionStreamResponse, ChatMessage, DeltaMessage,
                       FunctionResponse, ToolCall)
from .serving_base import OpenAIServingBase
from .serving_completions import build_sampling_params
from .usage_processor import UsageProcessor
from .utils import finish_reason_type, matched_stop, to_chat_logprobs


class OpenAIServingChat(OpenAIServingBase):
    def __init__(self, tokenizer_manager, template_manager):
        super().__init__(tokenizer_manager)
        self.template_manager = template_manager
        sa = tokenizer_manager.server_args
        self.tool_call_parser = sa.tool_call_parser
        self.reasoning_parser = sa.reasoning_parser

    def _validate_request(self, request: ChatCompletionRequest):
        if not request.messages:
            return "Messages cannot be empty."
        if isinstance(request.tool_choice, str) and request.tool_choice == "required" and not request.tools:
            return "Tools cannot be empty if tool choice is set to required."
        return None

    def _convert_to_internal_request(self, request: ChatCompletionRequest):
        tm = self.tokenizer_manager
        messages = []
        for m in request.messages:
            d = m.model_dump(exclude_none=True)
            if self.template_manager.jinja_template_content_format == "string":
                d["content"] = flatten_content(d.get("content"))
            if d.get("tool_calls"):
                for tc in d["tool_calls"]:
                    args = tc["function"].get("arguments")
                    if isinstance(args, str):
                        try:
                            tc["function"]["arguments"] = json.loads(args)
                        except Exception:
                            pass
            messages.append(d)
        tools = [t.model_dump() for t in request.tools] if request.tools and request.tool_choice != "none" else None
        kwargs = dict(request.chat_template_kwargs or {})
        if request.reasoning_effort:
            kwargs.setdefault("reasoning_effort", request.reasoning_effort)
        add_gen = True
        if request.continue_final_message and messages and messages[-1]["role"] == "assistant":
            add_gen = False
            kwargs["continue_final_message"] = True
        input_ids = self.template_manager.apply(tm.tokenizer, messages, tools, add_gen, **kwargs)
        stop = request.stop
        sp = build_sampling_params(request, stop=stop,
                                   max_new_tokens=request.max_completion_tokens or request.max_tokens)
        if sp["max_new_tokens"] is None:
            sp["max_new_tokens"] = max(tm.context_len - len(input_ids) - 1, 1)
        # tool constraints
        if tools and self.tool_call_parser and request.tool_choice != "auto":
            parser = FunctionCallParser(request.tools, self.tool_call_parser)
            c = parser.get_structure_constraint(request.tool_choice)
            if c is not None:
                kind, spec = c
                sp["ebnf" if kind == "ebnf" else "structural_tag"] = spec
        adapted = GenerateReqInput(
            input_ids=input_ids, sampling_params=sp, return_logprob=bool(request.logprobs),
            top_logprobs_num=request.top_logprobs or 0, logprob_start_len=-1, return_text_in_logprobs=True,
            stream=request.stream, lora_path=request.lora_path, rid=request.rid, extra_key=request.extra_key,
            return_hidden_states=request.return_hidden_states, return_routed_experts=request.return_routed_experts,
            bootstrap_host=request.bootstrap_host, bootstrap_port=request.bootstrap_port,
            bootstrap_room=request.bootstrap_room)
        return adapted, request

    # ------------------------------------------------------------------ non-streaming
    async def _handle_non_streaming_request(self, adapted, request, raw_request):
        ret = await self.tokenizer_manager.generate_request(adapted, raw_request).__anext__()
        if not isinstance(ret, list):
            ret = [ret]
        choices = []
        for idx, item in enumerate(ret):
            text = item["text"]
            reasoning = None
            if self.reasoning_parser and request.separate_reasoning:
                reasoning, text = ReasoningParser(self.reasoning_parser, False).parse_non_stream(text)
            tool_calls = None
            fr = item["meta_info"]["finish_reason"]
            fr_type = finish_reason_type(fr)
            if request.tools and request.tool_choice != "none" and self.tool_call_parser:
                parser = FunctionCallParser(request.tools, self.tool_call_parser)
                if parser.has_tool_call(text):
                    text, calls = parser.parse_non_stream(text)
                    if calls:
                        tool_calls = [ToolCall(id=f"call_{uuid.uuid4().hex[:24]}", index=c.tool_index,
                                               function=FunctionResponse(name=c.name, arguments=c.parameters))
                                      for c in calls]
                        if fr_type == "stop":
                            fr_type = "tool_calls"
            lp = None
            if request.logprobs:
                mi = item["meta_info"]
                lp = to_chat_logprobs(mi.get("output_token_logprobs"), mi.get("output_top_logprobs"))
            choices.append(ChatCompletionResponseChoice(
                index=idx, message=ChatMessage(role="assistant", content=text or None, reasoning_content=reasoning or None,
                                               tool_calls=tool_calls),
                logprobs=lp, finish_reason=fr_type, matched_stop=matched_stop(fr),
                hidden_states=item["meta_info"].get("hidden_states")))
        usage = UsageProcessor.calculate_response_usage(ret, request.n, self.tokenizer_manager.server_args.enable_cache_report)
        return ChatCompletionResponse(id=ret[0]["meta_info"]["id"], created=int(time.time()), model=request.model,
                                      choices=choices, usage=usage)

    # ------------------------------------------------------------------ streaming
    async def _generate_stream(self, adapted, request, raw_request):
        created = int(time.time())
        is_first, buffers, n_prev = {}, {}, {}
        prompt_tokens, completion_tokens, cached_tokens = {}, {}, {}
        reasoning_parsers, tool_parsers, has_tool = {}, {}, {}
        mi = {"id": ""}
        try:
            async for content in self.tokenizer_manager.generate_request(adapted, raw_request):
                index = content.get("index", 0)
                mi = content["meta_info"]
                prompt_tokens[index] = mi["prompt_tokens"]
                completion_tokens[index] = mi["completion_tokens"]
                cached_tokens[index] = mi.get("cached_tokens", 0)
                fr = mi["finish_reason"]
                if is_first.get(index, True):
                    is_first[index] = False
                    first = ChatCompletionStreamResponse(
                        id=mi["id"], created=created, model=request.model,
                        choices=[ChatCompletionResponseStreamChoice(index=index, delta=DeltaMessage(role="assistant", content=""))])
                    yield f"data: {first.model_dump_json()}\n\n"
                buf = buffers.get(index, "")
                delta = content["text"][len(buf):]
                buffers[index] = buf + delta
                lp = None
                if request.logprobs:
                    k = n_prev.get(index, 0)
                    lp = to_chat_logprobs(mi.get("output_token_logprobs", [])[k:], (mi.get("output_top_logprobs") or [])[k:])
                    n_prev[index] = len(mi.get("output_token_logprobs", []))
                if self.reasoning_parser and request.separate_reasoning and delta:
                    rp = reasoning_parsers.setdefault(index, ReasoningParser(self.reasoning_parser, request.stream_reasoning))
                    reasoning_delta, delta = rp.parse_stream_chunk(delta)
                    if reasoning_delta:
                        chunk = ChatCompletionStreamResponse(
                            id=mi["id"], created=created, model=request.model,
                            choices=[ChatCompletionResponseStreamChoice(index=index, delta=DeltaMessage(reasoning_content=reasoning_delta))])
                        yield f"data: {chunk.model_dump_json()}\n\n"
                if request.tools and request.tool_choice != "none" and self.tool_call_parser and delta:
                    tp = tool_parsers.setdefault(index, FunctionCallParser(request.tools, self.tool_call_parser))
                    delta, calls = tp.parse_stream_chunk(delta)
                    for c in calls:
                        has_tool[index] = True
                        tc = ToolCall(id=f"call_{uuid.uuid4().hex[:24]}" if c.name else None, index=c.tool_index,
                                      function=FunctionResponse(name=c.name, arguments=c.parameters))
                        chunk = ChatCompletionStreamResponse(
                            id=mi["id"], created=created, model=request.model,
                            choices=[ChatCompletionResponseStreamChoice(index=index, delta=DeltaMessage(tool_calls=[tc]))])
                        yield f"data: {chunk.model_dump_json()}\n\n"
                if delta or fr is not None:
                    fr_type = finish_reason_type(fr)
                    if fr_type == "stop" and has_tool.get(index):
                        fr_type = "tool_calls"
                    chunk = ChatCompletionStreamResponse(
                        id=mi["id"], created=created, model=request.model,
                        choices=[ChatCompletionResponseStreamChoice(index=index, delta=DeltaMessage(content=delta or None),
                                                                    logprobs=lp, finish_reason=fr_type,
                                                                    matched_stop=matched_stop(fr))])
                    yield f"data: {chunk.model_dump_json()}\n\n"
            if request.stream_options and request.stream_options.include_usage:
                usage = UsageProcessor.calculate_streaming_usage(prompt_tokens, completion_tokens, cached_tokens, request.n,
                                                                 self.tokenizer_manager.server_args.enable_cache_report)
                final = ChatCompletionStreamResponse(id=mi["id"], created=created, model=request.model, choices=[], usage=usage)
                yield f"data: {final.model_dump_json()}\n\n"
        except Exception as e:
            yield f"data: {self.create_streaming_error_response(str(e))}\n\n"
        yield "data: [DONE]\n\n"
