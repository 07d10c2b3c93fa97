"""OpenAI-compatible request / response models (reference
`python/sgl_jax/srt/entrypoints/openai/protocol.py:10-592`)."""

from __future__ import annotations

import time
import uuid
from typing import Any, Literal

from pydantic import BaseModel, Field


class ModelCard(BaseModel):
    id: str
    object: str = "model"
    created: int = Field(default_factory=lambda: int(time.time()))
    owned_by: str = "sglang"
    root: str | None = None
    max_model_len: int | None = None


class ModelList(BaseModel):
    object: str = "list"
    data: list[ModelCard] = Field(default_factory=list)


class ErrorResponse(BaseModel):
    object: str = "error"
    message: str
    type: str
    param: str | None = None
    code: int


class LogProbs(BaseModel):
    text_offset: list[int] = Field(default_factory=list)
    token_logprobs: list[float | None] = Field(default_factory=list)
    tokens: list[str] = Field(default_factory=list)
    top_logprobs: list[dict[str, float] | None] = Field(default_factory=list)


class TopLogprob(BaseModel):
    token: str
    bytes: list[int] | None = None
    logprob: float


class ChatCompletionTokenLogprob(BaseModel):
    token: str
    bytes: list[int] | None = None
    logprob: float
    top_logprobs: list[TopLogprob] = Field(default_factory=list)


class ChoiceLogprobs(BaseModel):
    content: list[ChatCompletionTokenLogprob] = Field(default_factory=list)


class UsageInfo(BaseModel):
    prompt_tokens: int = 0
    total_tokens: int = 0
    completion_tokens: int | None = 0
    prompt_tokens_details: dict[str, int] | None = None
    reasoning_tokens: int | None = 0


class StreamOptions(BaseModel):
    include_usage: bool | None = False
    continuous_usage_stats: bool | None = False


class JsonSchemaResponseFormat(BaseModel):
    name: str
    description: str | None = None
    schema_: dict[str, Any] | None = Field(alias="schema", default=None)
    strict: bool | None = False


class ResponseFormat(BaseModel):
    type: Literal["text", "json_object", "json_schema"]
    json_schema: JsonSchemaResponseFormat | None = None


class StructuresResponseFormat(BaseModel):
    begin: str
    schema_: dict[str, Any] | None = Field(alias="schema", default=None)
    end: str


class StructuralTagResponseFormat(BaseModel):
    type: Literal["structural_tag"]
    structures: list[StructuresResponseFormat]
    triggers: list[str]


class _SamplingExtras(BaseModel):
    # extensions shared by completions and chat completions
    top_k: int = -1
    min_p: float = 0.0
    min_tokens: int = 0
    json_schema: str | None = None
    regex: str | None = None
    ebnf: str | None = None
    repetition_penalty: float = 1.0
    stop_token_ids: list[int] | None = None
    no_stop_trim: bool = False
    ignore_eos: bool = False
    skip_special_tokens: bool = True
    lora_path: str | list[str | None] | None = None
    session_params: dict | None = None
    return_hidden_states: bool = False
    return_routed_experts: bool = False
    rid: str | list[str] | None = None
    extra_key: str | list[str] | None = None
    sampling_seed: int | None = None
    bootstrap_host: str | list[str] | None = None
    bootstrap_port: int | list[int | None] | None = None
    bootstrap_room: int | list[int] | None = None


class CompletionRequest(_SamplingExtras):
    model: str = "default"
    prompt: list[int] | list[list[int]] | str | list[str]
    best_of: int | None = None
    echo: bool = False
    frequency_penalty: float = 0.0
    logit_bias: dict[str, float] | None = None
    logprobs: int | None = None
    max_tokens: int | None = 16
    n: int = 1
    presence_penalty: float = 0.0
    seed: int | None = None
    stop: str | list[str] | None = None
    stream: bool = False
    stream_options: StreamOptions | None = None
    suffix: str | None = None
    temperature: float = 1.0
    top_p: float = 1.0
    user: str | None = None
    response_format: ResponseFormat | StructuralTagResponseFormat | None = None


class CompletionResponseChoice(BaseModel):
    index: int
    text: str
    logprobs: LogProbs | None = None
    finish_reason: Literal["stop", "length", "content_filter", "abort"] | None = None
    matched_stop: None | int | str = None
    hidden_states: Any = None


class CompletionResponse(BaseModel):
    id: str
    object: str = "text_completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str
    choices: list[CompletionResponseChoice]
    usage: UsageInfo
    metadata: dict[str, Any] | None = None


class CompletionResponseStreamChoice(CompletionResponseChoice):
    pass


class CompletionStreamResponse(BaseModel):
    id: str
    object: str = "text_completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str
    choices: list[CompletionResponseStreamChoice]
    usage: UsageInfo | None = None


class ChatCompletionMessageContentTextPart(BaseModel):
    type: Literal["text"]
    text: str


class ChatCompletionMessageContentImageURL(BaseModel):
    url: str
    detail: Literal["auto", "low", "high"] | None = "auto"


class ChatCompletionMessageContentImagePart(BaseModel):
    type: Literal["image_url"]
    image_url: ChatCompletionMessageContentImageURL | None = None


class FunctionResponse(BaseModel):
    name: str | None = None
    arguments: str | None = None


class ToolCall(BaseModel):
    id: str | None = None
    index: int | None = None
    type: Literal["function"] = "function"
    function: FunctionResponse


class ChatCompletionMessageGenericParam(BaseModel):
    role: Literal["system", "assistant", "tool", "function", "developer"]
    content: str | list[ChatCompletionMessageContentTextPart] | None = None
    tool_call_id: str | None = None
    name: str | None = None
    reasoning_content: str | None = None
    tool_calls: list[ToolCall] | None = None


class ChatCompletionMessageUserParam(BaseModel):
    role: Literal["user"]
    content: str | list[ChatCompletionMessageContentTextPart | ChatCompletionMessageContentImagePart]


ChatCompletionMessageParam = ChatCompletionMessageGenericParam | ChatCompletionMessageUserParam


class Function(BaseModel):
    description: str | None = None
    name: str | None = None
    parameters: dict | None = None
    strict: bool = False


class Tool(BaseModel):
    type: str = "function"
    function: Function


class ToolChoiceFuncName(BaseModel):
    name: str | None = None


class ToolChoice(BaseModel):
    function: ToolChoiceFuncName
    type: Literal["function"] = "function"


class ChatCompletionRequest(_SamplingExtras):
    messages: list[ChatCompletionMessageParam]
    model: str = "default"
    frequency_penalty: float = 0.0
    logit_bias: dict[str, float] | None = None
    logprobs: bool = False
    top_logprobs: int | None = None
    max_tokens: int | None = None
    max_completion_tokens: int | None = None
    n: int = 1
    presence_penalty: float = 0.0
    response_format: ResponseFormat | StructuralTagResponseFormat | None = None
    seed: int | None = None
    stop: str | list[str] | None = None
    stream: bool = False
    stream_options: StreamOptions | None = None
    temperature: float = 0.7
    top_p: float = 1.0
    user: str | None = None
    tools: list[Tool] | None = None
    tool_choice: ToolChoice | Literal["auto", "required", "none"] = "auto"
    return_hidden_states: bool = False
    reasoning_effort: Literal["low", "medium", "high"] | None = None
    continue_final_message: bool = False
    separate_reasoning: bool = True
    stream_reasoning: bool = True
    chat_template_kwargs: dict | None = None


class ChatMessage(BaseModel):
    role: str | None = None
    content: str | None = None
    reasoning_content: str | None = None
    tool_calls: list[ToolCall] | None = None


class ChatCompletionResponseChoice(BaseModel):
    index: int
    message: ChatMessage
    logprobs: LogProbs | ChoiceLogprobs | None = None
    finish_reason: Literal["stop", "length", "tool_calls", "content_filter", "function_call", "abort"] | None = None
    matched_stop: None | int | str = None
    hidden_states: Any = None


class ChatCompletionResponse(BaseModel):
    id: str
    object: str = "chat.completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str
    choices: list[ChatCompletionResponseChoice]
    usage: UsageInfo
    metadata: dict[str, Any] | None = None


class DeltaMessage(BaseModel):
    role: str | None = None
    content: str | None = None
    reasoning_content: str | None = None
    tool_calls: list[ToolCall] | None = None


class ChatCompletionResponseStreamChoice(BaseModel):
    index: int
    delta: DeltaMessage
    logprobs: LogProbs | ChoiceLogprobs | None = None
    finish_reason: Literal["stop", "length", "tool_calls", "content_filter", "function_call", "abort"] | None = None
    matched_stop: None | int | str = None


class ChatCompletionStreamResponse(BaseModel):
    id: str
    object: str = "chat.completion.chunk"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str
    choices: list[ChatCompletionResponseStreamChoice]
    usage: UsageInfo | None = None


class EmbeddingRequest(BaseModel):
    input: list[int] | list[list[int]] | str | list[str]
    model: str = "default"
    encoding_format: str = "float"
    dimensions: int | None = None
    user: str | None = None
    rid: str | list[str] | None = None


class EmbeddingObject(BaseModel):
    embedding: list[float]
    index: int
    object: str = "embedding"


class EmbeddingResponse(BaseModel):
    data: list[EmbeddingObject]
    model: str
    object: str = "list"
    usage: UsageInfo | None = None


class ScoringRequest(BaseModel):
    query: str | list[int] | None = None
    items: str | list[str] | list[list[int]] | None = None
    label_token_ids: list[int] | None = None
    apply_softmax: bool = False
    item_first: bool = False
    model: str = "default"


class ScoringResponse(BaseModel):
    scores: list[list[float]]
    model: str
    usage: UsageInfo | None = None
    object: str = "scoring"


class V1RerankReqInput(BaseModel):
    query: str
    documents: list[str]


class RerankResponse(BaseModel):
    score: float
    document: str
    index: int
    meta_info: dict | None = None


def random_id(prefix: str) -> str:
    return f"{prefix}-{uuid.uuid4().hex}"
