"""HTTP / OpenAI surface over a CPU engine (FastAPI TestClient), server-args parity, parsers."""

import dataclasses
import json

import pytest

from sglang_jax_b200.server_args import PortArgs, ServerArgs


@pytest.fixture(scope="module")
def client(tmp_path_factory):
    from fastapi.testclient import TestClient

    from sglang_jax_b200 import Engine
    from sglang_jax_b200.entrypoints.http_server import build_app_for_engine
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import write_tiny_qwen3_checkpoint
    ps.reset_state()
    path = write_tiny_qwen3_checkpoint(str(tmp_path_factory.mktemp("tiny")))
    eng = Engine(model_path=path, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                 max_total_tokens=8192, enable_single_process=True)
    with TestClient(build_app_for_engine(eng)) as c:
        yield c
    eng.shutdown()


def test_health_and_info(client):
    assert client.get("/health").status_code == 200
    assert client.get("/ping").status_code == 200
    assert client.get("/health_generate").status_code == 200
    info = client.get("/get_server_info").json()
    assert info["page_size"] == 16 and "internal_states" in info and info["max_total_num_tokens"] > 0
    assert client.get("/v1/models").json()["data"][0]["object"] == "model"
    assert client.get("/v1/models/nope").status_code == 404


def test_generate_native_and_stream(client):
    body = {"input_ids": [5, 6, 7, 8], "sampling_params": {"max_new_tokens": 5, "temperature": 0}}
    r = client.post("/generate", json=body).json()
    assert len(r["output_ids"]) == 5 and r["meta_info"]["finish_reason"]["type"] == "length"
    with client.stream("POST", "/generate", json={**body, "stream": True}) as s:
        lines = [l for l in s.iter_lines() if l]
    assert lines[-1] == "data: [DONE]"
    last = json.loads(lines[-2][6:])
    assert last["output_ids"] == r["output_ids"]
    # batch + logprobs
    r = client.post("/generate", json={"input_ids": [[1, 2, 3], [4, 5, 6, 7]], "return_logprob": True,
                                       "top_logprobs_num": 2, "logprob_start_len": 0,
                                       "sampling_params": {"max_new_tokens": 3, "temperature": 0}}).json()
    assert len(r) == 2
    m = r[1]["meta_info"]
    assert len(m["output_token_logprobs"]) == 3 and len(m["input_token_logprobs"]) == 4
    assert m["input_token_logprobs"][0][0] is None and len(m["output_top_logprobs"][0]) == 2


def test_openai_completions(client):
    r = client.post("/v1/completions", json={"model": "m", "prompt": [1, 2, 3, 4], "max_tokens": 4, "temperature": 0,
                                             "logprobs": 1})
    assert r.status_code == 200
    j = r.json()
    assert j["usage"]["completion_tokens"] == 4 and j["choices"][0]["finish_reason"] == "length"
    assert len(j["choices"][0]["logprobs"]["token_logprobs"]) == 4
    r = client.post("/v1/completions", json={"model": "m", "prompt": [1, 2, 3], "max_tokens": 3, "temperature": 0,
                                             "stream": True, "stream_options": {"include_usage": True}})
    chunks = [json.loads(l[6:]) for l in r.text.splitlines() if l.startswith("data: {")]
    assert chunks[-1]["usage"]["completion_tokens"] == 3
    assert client.post("/v1/completions", json={"model": "m", "prompt": []}).status_code == 400


def test_control_endpoints(client):
    assert client.post("/flush_cache").status_code == 200
    assert client.post("/pause_generation", json={"mode": "in_place"}).json()["status"] == "ok"
    assert client.post("/continue_generation").json()["status"] == "ok"
    assert client.post("/abort_request", json={"abort_all": True}).status_code == 200
    assert client.get("/get_load").json()[0]["num_reqs"] == 0
    assert client.post("/start_trace").status_code == 400       # tracer not enabled
    assert client.post("/release_memory_occupation").status_code == 501
    r = client.post("/separate_reasoning", json={"text": "<think>a</think>b", "reasoning_parser": "qwen3"}).json()
    assert r == {"reasoning_text": "a", "text": "b"}
    r = client.post("/parse_function_call", json={
        "text": '<tool_call>\n{"name": "f", "arguments": {"x": 1}}\n</tool_call>', "tool_call_parser": "qwen25",
        "tools": [{"type": "function", "function": {"name": "f", "parameters": {}}}]}).json()
    assert r["calls"][0]["name"] == "f" and json.loads(r["calls"][0]["parameters"]) == {"x": 1}


def test_input_too_long_is_400(client):
    r = client.post("/generate", json={"input_ids": list(range(5000)), "sampling_params": {"max_new_tokens": 4}})
    assert r.status_code == 400


# ---------------------------------------------------------------------------------- server args
REFERENCE_FIELDS = """model_path tokenizer_path tokenizer_mode tokenizer_backend skip_tokenizer_init load_format
model_loader_extra_config trust_remote_code context_length is_embedding revision model_impl model_layer_nums host port
skip_server_warmup warmups dtype quantization quantization_param_path quantization_config_path kv_cache_dtype
dtype_config mem_fraction_static max_running_requests max_total_tokens max_prefill_tokens chunked_prefill_size
enable_mixed_chunk schedule_policy schedule_conservativeness page_size swa_full_tokens_ratio
recurrent_state_memory_ratio max_recurrent_state_size recurrent_track_interval disable_hybrid_swa_memory device
device_indexes pd_disaggregation pd_prefill_mem_fraction pd_decode_mem_fraction pd_prefill_max_tokens
pd_decode_max_tokens pd_num_prefill pd_num_decode pd_prefill_tp_size pd_prefill_ep_size tp_size ep_size
ep_num_redundant_experts ep_dispatch_algorithm enable_sequence_parallel stream_interval stream_output random_seed
constrained_json_whitespace_pattern constrained_json_disable_any_whitespace watchdog_timeout dist_timeout download_dir
sleep_on_idle dp_size dp_schedule_policy log_level log_level_http log_requests log_requests_level crash_dump_folder
show_time_cost enable_metrics bucket_time_to_first_token bucket_inter_token_latency bucket_e2e_request_latency
decode_log_interval enable_request_time_stats_logging kv_events_config api_key served_model_name file_storage_path
enable_cache_report reasoning_parser tool_call_parser dist_init_addr nnodes node_rank json_model_override_args
preferred_sampling_params disable_radix_cache enable_unified_radix_tree hicache_storage hicache_ratio
hicache_write_through_threshold hicache_write_policy enable_recurrent_extra_buffer allow_auto_truncate
enable_tokenizer_batch_encode disable_overlap_schedule enable_precision_tracer attention_backend gdn_prefill_impl
dsa_use_pallas moe_backend disable_jax_allreduce_metadata enable_topk_kernel grammar_backend max_seq_len
precompile_token_paddings precompile_bs_paddings disable_precompile speculative_algorithm
speculative_draft_model_path speculative_draft_model_revision speculative_num_steps speculative_eagle_topk
speculative_num_draft_tokens speculative_accept_threshold_single speculative_accept_threshold_acc
enable_deterministic_sampling enable_single_process enable_nan_detection use_sort_for_toppk_minp enable_lora
max_lora_rank lora_target_modules lora_paths max_loaded_loras max_loras_per_batch lora_eviction_policy
enable_static_lora lora_scaling enable_engine_loop_run_forever_daemon multimodal enable_return_routed_experts
enable_expert_balance_debug expert_balance_segment_counter expert_balance_output_file init_expert_location
enable_expert_distribution_recorder expert_distribution_recorder_buffer_size
expert_distribution_recorder_output_file disaggregation_mode disaggregation_bootstrap_url
disaggregation_bootstrap_port disaggregation_transfer_port disaggregation_enable_d2h disaggregation_use_raiden
disaggregation_enable_chunk_prefill_transfer disaggregation_side_channel_port disaggregation_d2h_pool_size
disaggregation_d2h_max_tokens disaggregation_channel_number disaggregation_host_ip
disaggregation_bootstrap_timeout_seconds disaggregation_pull_timeout_seconds disaggregation_ack_timeout_seconds
disaggregation_orphan_reaper_interval_seconds disaggregation_shared_secret disaggregation_decode_watchdog_seconds
disaggregation_num_reserved_decode_tokens disaggregation_max_inflight_transfers""".split()


def test_server_args_flag_parity_and_defaults():
    names = {f.name for f in dataclasses.fields(ServerArgs)}
    missing = [f for f in REFERENCE_FIELDS if f not in names]
    assert not missing, missing
    a = ServerArgs(model_path="m", device="cpu")
    assert (a.mem_fraction_static, a.chunked_prefill_size, a.random_seed, a.schedule_policy, a.page_size,
            a.max_prefill_tokens, a.watchdog_timeout, a.stream_interval, a.grammar_backend) == \
        (0.88, 4096, 42, "fcfs", 1, 16384, 300, 1, "llguidance")
    assert a.dp_schedule_policy == "cache_aware"
    assert ServerArgs(model_path="m", device="cpu", disable_radix_cache=True).dp_schedule_policy == "round_robin"
    b = ServerArgs.from_cli(["--model-path", "m", "--tp", "4", "--dp-size", "2", "--device", "cpu", "--page-size", "64",
                             "--chunked-prefill-size", "8192", "--enable-mixed-chunk", "--lora-paths", "a", "b"])
    assert b.tp_size == 4 and b.tensor_size == 2 and b.enable_mixed_chunk and b.lora_paths == ["a", "b"] and b.enable_lora
    # a bare --pd-disaggregation selects the in-node launcher, like the reference's bare flag selects its split
    assert ServerArgs.from_cli(["--model-path", "m", "--pd-disaggregation", "--page-size", "16"]).pd_disaggregation == "local"
    assert ServerArgs.from_cli(["--model-path", "m", "--pd-disaggregation", "pathways", "--page-size", "16"]
                               ).pd_disaggregation == "pathways"
    assert ServerArgs.from_cli(["--model-path", "m"]).pd_disaggregation == ""
    with pytest.raises(AssertionError):
        ServerArgs(model_path="m", device="cpu", page_size=48, chunked_prefill_size=100)
    with pytest.raises(AssertionError):
        ServerArgs(model_path="m", device="cpu", tp_size=3, nnodes=2)
    p = PortArgs.init_new(a)
    assert p.tokenizer_ipc_name.startswith("ipc://") and p.pub_sub_addr is None


# ---------------------------------------------------------------------------------- parsers
TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}, "required": ["city"]}}}]


@pytest.mark.parametrize("parser,text", [
    ("qwen25", 'Sure.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris", "days": 3}}\n</tool_call>'),
    ("qwen3_coder", "Sure.\n<tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n"
                    "<parameter=days>\n3\n</parameter>\n</function>\n</tool_call>"),
    ("glm45", "Sure.\n<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Paris</arg_value>\n"
              "<arg_key>days</arg_key>\n<arg_value>3</arg_value>\n</tool_call>"),
    ("mimo", 'Sure.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris", "days": 3}}\n</tool_call>'),
])
def test_function_call_parsers_stream_equals_non_stream(parser, text):
    from sglang_jax_b200.function_call.function_call_parser import FunctionCallParser
    normal, calls = FunctionCallParser(TOOLS, parser).parse_non_stream(text)
    assert normal == "Sure." and calls[0].name == "get_weather"
    assert json.loads(calls[0].parameters) == {"city": "Paris", "days": 3}
    p = FunctionCallParser(TOOLS, parser)
    name, args, normal_s = None, "", ""
    for i in range(0, len(text), 5):
        n, cs = p.parse_stream_chunk(text[i:i + 5])
        normal_s += n
        for c in cs:
            name = c.name or name
            args += c.parameters
    assert name == "get_weather" and json.loads(args) == {"city": "Paris", "days": 3}
    assert normal_s.strip() == "Sure."


def test_undefined_function_is_dropped_and_ebnf_built():
    from sglang_jax_b200.function_call.function_call_parser import FunctionCallParser
    p = FunctionCallParser(TOOLS, "qwen25")
    normal, calls = p.parse_non_stream('<tool_call>\n{"name": "nope", "arguments": {}}\n</tool_call>')
    assert calls == []
    kind, spec = p.get_structure_constraint("required")
    assert kind == "ebnf" and "get_weather" in spec and spec.startswith("root ::=")


def test_reasoning_parser_streaming():
    from sglang_jax_b200.reasoning_parser import ReasoningParser
    p = ReasoningParser("qwen3")
    r = n = ""
    for c in ["<th", "ink>I am ", "thinking</th", "ink>\n\nThe ans", "wer"]:
        a, b = p.parse_stream_chunk(c)
        r += a
        n += b
    assert r == "I am thinking" and n == "The answer"
    assert ReasoningParser("deepseek-r1").parse_non_stream("abc</think>x") == ("abc", "x")
    with pytest.raises(ValueError):
        ReasoningParser("unknown-model")


def test_profile_endpoints_honour_name_and_activities(client, tmp_path):
    """`/start_profile` with a run name and an activity list (what `python -m sglang_jax_b200.profiler --profile-name
    ... --no-gpu --mem` sends): the trace file carries the name; stop is refused when nothing runs."""
    import glob
    out = str(tmp_path / "prof")
    r = client.post("/start_profile", json={"output_dir": out, "profile_name": "run-a", "activities": ["CPU", "MEM"]})
    assert r.status_code == 200
    assert client.get("/profile_status").status_code == 200
    client.post("/generate", json={"input_ids": [5, 6, 7], "sampling_params": {"max_new_tokens": 3, "temperature": 0}})
    assert client.post("/stop_profile").status_code == 200
    assert glob.glob(out + "/run-a*-TP-0.trace.json.gz")
    assert client.post("/stop_profile").status_code != 200
