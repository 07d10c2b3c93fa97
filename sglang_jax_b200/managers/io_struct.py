"""Messages exchanged between the front-end (HTTP / Engine + TokenizerManager), the
Scheduler and the DetokenizerManager.

The set of message types and their field names match the reference's
`python/sgl_jax/srt/managers/io_struct.py:30-845` so that code written against
`GenerateReqInput` / `BatchTokenIDOut` keeps working; they travel as pickles over
ZMQ PUSH/PULL sockets, or over in-process queues in single-process mode.
"""

from __future__ import annotations

import copy
import uuid
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Literal


@dataclass
class BaseReq:
    rid: str | list[str] | None = field(default=None, kw_only=True)
    http_worker_ipc: str | None = field(default=None, kw_only=True)

    def regenerate_rid(self):
        if isinstance(self.rid, list):
            self.rid = [uuid.uuid4().hex for _ in self.rid]
        else:
            self.rid = uuid.uuid4().hex
        return self.rid


@dataclass
class GenerateReqInput:
    """A user-level generation request: one prompt or a batch of prompts."""

    text: list[str] | str | None = None
    input_ids: list[list[int]] | list[int] | None = None
    input_embeds: Any = None
    image_data: Any = None
    video_data: Any = None
    audio_data: Any = None
    # per request: {"input_embedding": [prompt_len, hidden], "mrope_positions": [3, prompt_len],
    # "mrope_position_delta": int} produced by an encoder stage (one dict, or a list for a batch)
    mm_inputs: list[dict] | dict | None = None
    sampling_params: list[dict] | dict | None = None
    rid: list[str] | str | None = None
    return_logprob: list[bool] | bool | None = None
    return_output_logprob_only: bool | None = None
    logprob_start_len: list[int] | int | None = None
    top_logprobs_num: list[int] | int | None = None
    token_ids_logprob: list[list[int]] | list[int] | None = None
    return_text_in_logprobs: bool = True
    stream: bool = False
    lora_path: list[str] | str | None = None
    lora_id: list[str] | str | None = None
    extra_key: list[str] | str | None = None
    return_routed_experts: list[bool] | bool | None = None
    return_hidden_states: bool = False
    dp_rank: list[int] | int | None = None
    bootstrap_host: list[str] | str | None = None
    bootstrap_port: list[int] | int | None = None
    bootstrap_room: list[int] | int | None = None
    disagg_prefill_dp_rank: list[int] | int | None = None
    disagg_transfer_id: list[str] | str | None = None
    # filled by normalize_batch_and_arguments
    batch_size: int = 1
    is_single: bool = True
    parallel_sample_num: int = 1

    def normalize_batch_and_arguments(self):
        if self.text is None and self.input_ids is None and self.input_embeds is None:
            raise ValueError("Either text, input_ids or input_embeds should be provided.")
        if sum(x is not None for x in (self.text, self.input_ids, self.input_embeds)) > 1:
            raise ValueError("Only one of text, input_ids, and input_embeds should be provided.")
        if self.text is not None:
            self.is_single = isinstance(self.text, str)
            self.batch_size = 1 if self.is_single else len(self.text)
        elif self.input_ids is not None:
            if len(self.input_ids) == 0:
                raise ValueError("input_ids cannot be empty.")
            self.is_single = isinstance(self.input_ids[0], int)
            self.batch_size = 1 if self.is_single else len(self.input_ids)
        else:
            self.is_single = not isinstance(self.input_embeds[0][0], list)
            self.batch_size = 1 if self.is_single else len(self.input_embeds)

        sp = self.sampling_params
        if sp is None:
            sp = {}
        if isinstance(sp, dict):
            self.parallel_sample_num = sp.get("n", 1)
        else:
            ns = {p.get("n", 1) for p in sp}
            if len(ns) > 1:
                raise ValueError("The parallel_sample_num should be the same for all samples in sample params.")
            self.parallel_sample_num = ns.pop() if ns else 1
        if self.parallel_sample_num > 1 and self.is_single:
            # n>1 on a single prompt is expanded as a batch of one.
            self.is_single = False
            if self.text is not None:
                self.text = [self.text]
            if self.input_ids is not None:
                self.input_ids = [self.input_ids]

        if self.is_single:
            self.sampling_params = sp if isinstance(sp, dict) else sp[0]
            if self.rid is None:
                self.rid = uuid.uuid4().hex
            if self.return_logprob is None:
                self.return_logprob = False
            if self.logprob_start_len is None:
                self.logprob_start_len = -1
            if self.top_logprobs_num is None:
                self.top_logprobs_num = 0
            if self.return_routed_experts is None:
                self.return_routed_experts = False
            return

        n = self.batch_size

        def per_item(v, default):
            if v is None:
                return [copy.copy(default) for _ in range(n)]
            if isinstance(v, list):
                if len(v) != n:
                    raise ValueError(f"per-request list has length {len(v)}, expected {n}")
                return v
            return [copy.copy(v) for _ in range(n)]

        if isinstance(sp, dict):
            self.sampling_params = [dict(sp) for _ in range(n)]
        else:
            self.sampling_params = per_item(sp, {})
        if self.rid is None:
            self.rid = [uuid.uuid4().hex for _ in range(n)]
        elif isinstance(self.rid, str):
            self.rid = [f"{self.rid}_{i}" for i in range(n)] if n > 1 else [self.rid]
        self.return_logprob = per_item(self.return_logprob, False)
        self.logprob_start_len = per_item(self.logprob_start_len, -1)
        self.top_logprobs_num = per_item(self.top_logprobs_num, 0)
        if self.token_ids_logprob is not None and self.token_ids_logprob and isinstance(self.token_ids_logprob[0], int):
            self.token_ids_logprob = [list(self.token_ids_logprob) for _ in range(n)]
        else:
            self.token_ids_logprob = per_item(self.token_ids_logprob, None)
        self.lora_path = per_item(self.lora_path, None)
        self.mm_inputs = per_item(self.mm_inputs, None)
        self.lora_id = per_item(self.lora_id, None)
        self.extra_key = per_item(self.extra_key, None)
        self.return_routed_experts = per_item(self.return_routed_experts, False)
        self.dp_rank = per_item(self.dp_rank, None)
        self.bootstrap_host = per_item(self.bootstrap_host, None)
        self.bootstrap_port = per_item(self.bootstrap_port, None)
        self.bootstrap_room = per_item(self.bootstrap_room, None)
        self.disagg_prefill_dp_rank = per_item(self.disagg_prefill_dp_rank, None)
        self.disagg_transfer_id = per_item(self.disagg_transfer_id, None)

    def __getitem__(self, i: int) -> "GenerateReqInput":
        def g(v):
            return v[i] if isinstance(v, list) else v

        return GenerateReqInput(
            text=self.text[i] if self.text is not None else None,
            input_ids=self.input_ids[i] if self.input_ids is not None else None,
            input_embeds=self.input_embeds[i] if self.input_embeds is not None else None,
            mm_inputs=g(self.mm_inputs),
            sampling_params=self.sampling_params[i],
            rid=self.rid[i],
            return_logprob=g(self.return_logprob),
            return_output_logprob_only=self.return_output_logprob_only,
            logprob_start_len=g(self.logprob_start_len),
            top_logprobs_num=g(self.top_logprobs_num),
            token_ids_logprob=self.token_ids_logprob[i] if self.token_ids_logprob else None,
            return_text_in_logprobs=self.return_text_in_logprobs,
            stream=self.stream,
            lora_path=g(self.lora_path), lora_id=g(self.lora_id), extra_key=g(self.extra_key),
            return_routed_experts=g(self.return_routed_experts),
            return_hidden_states=self.return_hidden_states,
            dp_rank=g(self.dp_rank),
            bootstrap_host=g(self.bootstrap_host), bootstrap_port=g(self.bootstrap_port),
            bootstrap_room=g(self.bootstrap_room),
            disagg_prefill_dp_rank=g(self.disagg_prefill_dp_rank),
            disagg_transfer_id=g(self.disagg_transfer_id),
        )


@dataclass
class VertexGenerateReqInput(GenerateReqInput):
    instances: list[dict] | None = None
    parameters: dict | None = None


@dataclass
class TokenizedGenerateReqInput:
    rid: str | None = None
    text: str | None = None
    input_ids: list[int] | None = None
    sampling_params: Any = None  # SamplingParams
    return_logprob: bool = False
    return_output_logprob_only: bool | None = None
    logprob_start_len: int = -1
    top_logprobs_num: int = 0
    token_ids_logprob: list[int] | None = None
    stream: bool = False
    lora_id: str | None = None
    extra_key: str | None = None
    return_routed_experts: bool = False
    return_hidden_states: bool = False
    mm_inputs: dict | None = None
    dp_rank: int | None = None
    bootstrap_host: str | None = None
    bootstrap_port: int | None = None
    bootstrap_room: int | None = None
    disagg_prefill_dp_rank: int | None = None
    disagg_transfer_id: str | None = None
    session_id: str | None = None


@dataclass
class EmbeddingReqInput:
    text: list[str] | str | None = None
    input_ids: list[list[int]] | list[int] | None = None
    rid: list[str] | str | None = None
    image_data: Any = None
    video_data: Any = None
    audio_data: Any = None
    normalize: bool = True
    extra_key: str | None = None
    is_single: bool = True
    batch_size: int = 1

    def normalize_batch_and_arguments(self):
        if self.text is None and self.input_ids is None:
            raise ValueError("Either text or input_ids should be provided.")
        if self.text is not None:
            self.is_single = isinstance(self.text, str)
            self.batch_size = 1 if self.is_single else len(self.text)
        else:
            self.is_single = isinstance(self.input_ids[0], int)
            self.batch_size = 1 if self.is_single else len(self.input_ids)
        if self.is_single:
            if self.rid is None:
                self.rid = uuid.uuid4().hex
        else:
            if self.rid is None:
                self.rid = [uuid.uuid4().hex for _ in range(self.batch_size)]

    def __getitem__(self, i):
        return EmbeddingReqInput(
            text=self.text[i] if self.text is not None else None,
            input_ids=self.input_ids[i] if self.input_ids is not None else None,
            rid=self.rid[i], normalize=self.normalize, extra_key=self.extra_key)


@dataclass
class TokenizedEmbeddingReqInput:
    rid: str
    text: str
    input_ids: list[int]
    normalize: bool = True
    extra_key: str | None = None


@dataclass
class BatchTokenIDOut:
    rids: list[str]
    finished_reasons: list[dict | None]
    decoded_texts: list[str]
    decode_ids: list[list[int]]
    read_offsets: list[int]
    output_ids: list[list[int]] | None
    skip_special_tokens: list[bool]
    spaces_between_special_tokens: list[bool]
    no_stop_trim: list[bool]
    prompt_tokens: list[int]
    completion_tokens: list[int]
    cached_tokens: list[int]
    input_token_logprobs_val: list = field(default_factory=list)
    input_token_logprobs_idx: list = field(default_factory=list)
    output_token_logprobs_val: list = field(default_factory=list)
    output_token_logprobs_idx: list = field(default_factory=list)
    input_top_logprobs_val: list = field(default_factory=list)
    input_top_logprobs_idx: list = field(default_factory=list)
    output_top_logprobs_val: list = field(default_factory=list)
    output_top_logprobs_idx: list = field(default_factory=list)
    input_token_ids_logprobs_val: list = field(default_factory=list)
    input_token_ids_logprobs_idx: list = field(default_factory=list)
    output_token_ids_logprobs_val: list = field(default_factory=list)
    output_token_ids_logprobs_idx: list = field(default_factory=list)
    output_hidden_states: list | None = None
    output_hidden_states_for_mm: list | None = None
    cache_miss_count: int | None = None
    output_routed_experts: list | None = None
    spec_verify_ct: list[int] | None = None
    dp_ranks: list[int] | None = None       # data-parallel section of each request (dp_size > 1 only)


@dataclass
class BatchStrOut:
    rids: list[str]
    finished_reasons: list[dict | None]
    output_strs: list[str]
    output_ids: list[list[int]] | None
    prompt_tokens: list[int]
    completion_tokens: list[int]
    cached_tokens: list[int]
    input_token_logprobs_val: list = field(default_factory=list)
    input_token_logprobs_idx: list = field(default_factory=list)
    output_token_logprobs_val: list = field(default_factory=list)
    output_token_logprobs_idx: list = field(default_factory=list)
    input_top_logprobs_val: list = field(default_factory=list)
    input_top_logprobs_idx: list = field(default_factory=list)
    output_top_logprobs_val: list = field(default_factory=list)
    output_top_logprobs_idx: list = field(default_factory=list)
    input_token_ids_logprobs_val: list = field(default_factory=list)
    input_token_ids_logprobs_idx: list = field(default_factory=list)
    output_token_ids_logprobs_val: list = field(default_factory=list)
    output_token_ids_logprobs_idx: list = field(default_factory=list)
    output_hidden_states: list | None = None
    cache_miss_count: int | None = None
    output_routed_experts: list | None = None
    spec_verify_ct: list[int] | None = None
    dp_ranks: list[int] | None = None       # data-parallel section of each request (dp_size > 1 only)


@dataclass
class BatchEmbeddingOut:
    rids: list[str]
    finished_reasons: list[dict | None]
    embeddings: list[list[float]]
    prompt_tokens: list[int]
    cached_tokens: list[int] = field(default_factory=list)


@dataclass
class AbortReq(BaseReq):
    abort_all: bool = False
    finished_reason: dict[str, Any] | None = None
    aborted_message: str | None = None


@dataclass
class PauseGenerationReqInput(BaseReq):
    """`abort`: finish every in-flight request with an abort reason.
    `in_place`: stop stepping, keep every request and its KV where it is.
    `retract`: stop stepping and move running requests back to the waiting queue,
    releasing their KV (they re-prefill on continue)."""
    mode: Literal["abort", "retract", "in_place"] = "abort"


@dataclass
class ContinueGenerationReqInput(BaseReq):
    pass


@dataclass
class FlushCacheReqInput(BaseReq):
    pass


@dataclass
class FlushCacheReqOutput(BaseReq):
    success: bool = True
    flushed_items: int = 0
    error_msg: str = ""


@dataclass
class RpcReqInput:
    request_id: str = ""


@dataclass
class RpcReqOutput:
    request_id: str = ""
    success: bool = True
    error_msg: str = ""


@dataclass
class ReleaseMemoryOccupationReqInput(RpcReqInput):
    memory_size: int = 0


@dataclass
class ResumeMemoryOccupationReqInput(RpcReqInput):
    memory_size: int = 0


@dataclass
class ReleaseMemoryOccupationReqOutput(RpcReqOutput):
    pass


@dataclass
class ResumeMemoryOccupationReqOutput(RpcReqOutput):
    pass


@dataclass
class OpenSessionReqInput(RpcReqInput):
    session_id: str = ""
    capacity_of_str_len: int = 0


@dataclass
class CloseSessionReqInput(RpcReqInput):
    session_id: str = ""


@dataclass
class OpenSessionReqOutput(RpcReqOutput):
    session_id: str = ""


@dataclass
class CloseSessionReqOutput(RpcReqOutput):
    pass


@dataclass
class ConfigureLoggingReq(RpcReqInput):
    log_level: str | None = None
    log_file: str | None = None
    log_requests: bool | None = None
    log_requests_level: int | None = None


@dataclass
class ConfigureLoggingReqOutput(RpcReqOutput):
    pass


@dataclass
class GetInternalStateReq:
    pass


@dataclass
class GetInternalStateReqOutput:
    internal_state: dict[Any, Any] = field(default_factory=dict)


@dataclass
class SetInternalStateReq(RpcReqInput):
    state_data: dict[str, Any] = field(default_factory=dict)


@dataclass
class SetInternalStateReqOutput(RpcReqOutput):
    updated: bool = True
    server_args: dict[str, Any] = field(default_factory=dict)


@dataclass
class GetLoadReqInput:
    pass


@dataclass
class GetLoadReqOutput:
    dp_rank: int = 0
    num_reqs: int = 0
    num_waiting_reqs: int = 0
    num_tokens: int = 0


@dataclass
class ProfileReqInput:
    output_dir: str | None = None
    start_step: int | None = None
    num_steps: int | None = None
    host_tracer_level: int | None = None
    python_tracer_level: int | None = None
    stage_id: int | None = None
    profile_by_stage: bool | None = False
    profile_stages: list[str] | None = None
    activities: list[str] | None = None      # subset of CPU, GPU, MEM (default CPU + GPU)
    profile_name: str | None = None          # file-name stem of the traces (default: a time stamp)


class ProfileReqType(Enum):
    START_PROFILE = 1
    STOP_PROFILE = 2
    STATUS = 3


@dataclass
class ProfileReq:
    type: ProfileReqType = ProfileReqType.START_PROFILE
    output_dir: str | None = None
    start_step: int | None = None
    num_steps: int | None = None
    host_tracer_level: int | None = None
    python_tracer_level: int | None = None
    profile_id: str | None = None
    stage_id: int | None = None
    profile_by_stage: bool | None = False
    profile_stages: list[str] | None = None
    activities: list[str] | None = None


@dataclass
class ProfileReqOutput:
    success: bool = True
    message: str = ""


@dataclass
class HealthCheckOutput:
    status: str = "healthy"
    timestamp: float = 0.0


@dataclass
class ParseFunctionCallReq(RpcReqInput):
    text: str = ""
    tools: list | None = None
    parser_type: str = "default"
    tool_call_parser: str | None = None


@dataclass
class SeparateReasoningReqInput(RpcReqInput):
    text: str = ""
    reasoning_type: str = "default"
    reasoning_parser: str | None = None


@dataclass
class StartTraceReqInput(RpcReqInput):
    req_num: int | None = None
    output_file: str | None = None
    save_tensor: bool = False


@dataclass
class StopTraceReqInput(RpcReqInput):
    pass


@dataclass
class TraceStatusReqInput(RpcReqInput):
    pass


@dataclass
class LoadLoRAAdapterReqInput(RpcReqInput):
    lora_name: str = ""
    lora_path: str = ""
    pinned: bool = False
    lora_id: str | None = None


@dataclass
class UnloadLoRAAdapterReqInput(RpcReqInput):
    lora_name: str = ""
    lora_id: str | None = None


@dataclass
class LoRAUpdateOutput(RpcReqOutput):
    loaded_adapters: dict[str, str] = field(default_factory=dict)


@dataclass
class SchedulerFailure:
    """Sent to the front end when the scheduler loop dies: every pending request fails."""
    message: str = ""
