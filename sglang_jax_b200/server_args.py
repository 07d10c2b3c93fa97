"""Server arguments: one dataclass that is at once the CLI, the `Engine(**kwargs)`
signature and the config snapshot handed to every subprocess.

Field names and defaults follow the reference's `ServerArgs`
(`python/sgl_jax/srt/server_args.py:54-298`) so that a launch line written for it
works here.  The CLI is *generated* from the dataclass (type, default, choices and
help come from field metadata) instead of being a hand-written argparse list, and
derived defaults are resolved in `__post_init__` (reference `:300-606`).
B200-specific additions are grouped at the end and are all optional.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import os
import random
import tempfile
from dataclasses import dataclass, field
from typing import Any, get_args, get_origin

SCHEDULE_POLICIES = ["lpm", "random", "fcfs", "dfs-weight", "lof"]
DP_SCHEDULE_POLICIES = ["round_robin", "min_running_queue", "cache_aware", "shape_aware"]
LOAD_FORMATS = [
    "auto", "pt", "safetensors", "npcache", "dummy", "random", "sharded_state", "gguf",
    "bitsandbytes", "mistral", "layered", "jax",
]
ATTENTION_BACKENDS = ["fa", "native", "sm100"]
MOE_BACKENDS = ["epmoe", "fused", "fused_v2", "auto"]
SPEC_ALGOS = [None, "EAGLE", "EAGLE3", "NEXTN", "STANDALONE", "DFLASH"]


def _m(help: str = "", choices=None, aliases=(), const=None) -> dict:
    return {"help": help, "choices": choices, "aliases": tuple(aliases), "const": const}


@dataclass
class ServerArgs:
    # --- model / tokenizer -------------------------------------------------
    model_path: str = field(default="", metadata=_m("HF repo id or local directory of the model"))
    tokenizer_path: str | None = None
    tokenizer_mode: str = field(default="auto", metadata=_m(choices=["auto", "slow"]))
    tokenizer_backend: str = field(default="huggingface", metadata=_m(choices=["huggingface", "fastokens", "tiktoken"]))
    skip_tokenizer_init: bool = False
    load_format: str = field(default="auto", metadata=_m(choices=LOAD_FORMATS))
    model_loader_extra_config: str = "{}"
    trust_remote_code: bool = False
    context_length: int | None = None
    is_embedding: bool = False
    revision: str | None = None
    model_impl: str = "auto"
    model_layer_nums: int | None = None
    # --- HTTP ----------------------------------------------------------------
    host: str = "127.0.0.1"
    port: int = 30000
    skip_server_warmup: bool = False
    warmups: str | None = None
    # --- dtype / quantization --------------------------------------------------
    dtype: str = field(default="auto", metadata=_m(choices=["auto", "half", "float16", "bfloat16", "float", "float32"]))
    quantization: str | None = None
    quantization_param_path: str | None = None
    quantization_config_path: str | None = None
    kv_cache_dtype: str = field(default="auto", metadata=_m(choices=["auto", "bf16", "bfloat16", "fp8_e4m3", "fp8_e5m2"]))
    dtype_config: str | None = None
    # --- memory / scheduling --------------------------------------------------
    mem_fraction_static: float | None = None
    max_running_requests: int | None = None
    max_total_tokens: int | None = None
    max_prefill_tokens: int = 16384
    chunked_prefill_size: int | None = None
    enable_mixed_chunk: bool = False
    schedule_policy: str = field(default="fcfs", metadata=_m(choices=SCHEDULE_POLICIES))
    schedule_conservativeness: float = 1.0
    page_size: int = 1
    swa_full_tokens_ratio: float = 0.8
    # hybrid linear-attention models: recurrent-state checkpoints kept for shared prefixes (0 = no sharing)
    recurrent_snapshot_slots: int = 32
    recurrent_state_memory_ratio: float = 0.9
    max_recurrent_state_size: int | None = None
    recurrent_track_interval: int | None = None
    disable_hybrid_swa_memory: bool = False
    # --- device ----------------------------------------------------------------
    device: str | None = None
    device_indexes: list[int] | None = None
    # --- PD disaggregation (launcher-level) --------------------------------------
    pd_disaggregation: str = field(default="", metadata=_m(
        const="local", help="in-node P/D split behind one front door: prefill and decode engines on slices of the "
                            "devices (`local`; `pathways`, the reference's name for its in-process split, is "
                            "accepted as a synonym)"))
    pd_prefill_mem_fraction: float = 0.85
    pd_decode_mem_fraction: float = 0.85
    pd_prefill_max_tokens: int = 20480
    pd_decode_max_tokens: int = 25600
    pd_num_prefill: int = 1
    pd_num_decode: int = 1
    pd_prefill_tp_size: int = 0
    pd_prefill_ep_size: int = 0
    # --- parallelism ---------------------------------------------------------------
    tp_size: int = field(default=1, metadata=_m("tensor-parallel size (total GPUs of one replica)", aliases=["--tp", "--tensor-parallel-size"]))
    ep_size: int = field(default=1, metadata=_m(aliases=["--ep", "--expert-parallel-size"]))
    ep_num_redundant_experts: int = 0
    ep_dispatch_algorithm: str | None = None
    enable_sequence_parallel: bool = False
    stream_interval: int = 1
    stream_output: bool = False
    random_seed: int | None = None
    constrained_json_whitespace_pattern: str | None = None
    constrained_json_disable_any_whitespace: bool = False
    watchdog_timeout: float = 300
    dist_timeout: int | None = None
    download_dir: str | None = None
    sleep_on_idle: bool = False
    dp_size: int = field(default=1, metadata=_m(aliases=["--dp", "--data-parallel-size"]))
    dp_schedule_policy: str | None = field(default=None, metadata=_m(choices=[None] + DP_SCHEDULE_POLICIES))
    # --- logging / metrics ------------------------------------------------------------
    log_level: str = "info"
    log_level_http: str | None = None
    log_requests: bool = False
    log_requests_level: int = field(default=0, metadata=_m(choices=[0, 1, 2, 3]))
    crash_dump_folder: str | None = None
    show_time_cost: bool = False
    enable_metrics: bool = False
    bucket_time_to_first_token: list[float] | None = None
    bucket_inter_token_latency: list[float] | None = None
    bucket_e2e_request_latency: list[float] | None = None
    decode_log_interval: int = 40
    enable_request_time_stats_logging: bool = False
    kv_events_config: str | None = None
    # --- API ---------------------------------------------------------------------------
    api_key: str | None = None
    served_model_name: str | None = None
    file_storage_path: str = "sglang_storage"
    enable_cache_report: bool = False
    reasoning_parser: str | None = None
    tool_call_parser: str | None = None
    # --- multi-node -----------------------------------------------------------------------
    dist_init_addr: str | None = None
    nnodes: int = 1
    node_rank: int = 0
    json_model_override_args: str = "{}"
    preferred_sampling_params: str | None = None
    # --- cache ------------------------------------------------------------------------------
    disable_radix_cache: bool = False
    enable_unified_radix_tree: bool = False
    hicache_storage: str = field(default="disable", metadata=_m(choices=["disable", "host"]))
    hicache_ratio: float = 2.0
    hicache_write_through_threshold: int = 1
    hicache_write_policy: str = field(default="write_through", metadata=_m(choices=["write_through", "write_back", "write_through_selective"]))
    enable_recurrent_extra_buffer: bool = False
    allow_auto_truncate: bool = False
    enable_tokenizer_batch_encode: bool = False
    disable_overlap_schedule: bool = False
    enable_precision_tracer: bool = False
    # --- kernels -----------------------------------------------------------------------------
    attention_backend: str = field(default="fa", metadata=_m("fa/sm100 = hand-written paged attention kernels; native = torch reference", choices=ATTENTION_BACKENDS))
    gdn_prefill_impl: str = "fused_chunk_parallel"
    dsa_use_pallas: bool = True
    moe_backend: str = field(default="epmoe", metadata=_m(choices=MOE_BACKENDS))
    disable_jax_allreduce_metadata: bool = False
    enable_topk_kernel: bool = True
    grammar_backend: str | None = None
    max_seq_len: int = 4096
    precompile_token_paddings: list[int] | None = None
    precompile_bs_paddings: list[int] | None = None
    disable_precompile: bool = False
    # --- speculative decoding -------------------------------------------------------------------
    speculative_algorithm: str | None = field(default=None, metadata=_m(choices=SPEC_ALGOS))
    speculative_draft_model_path: str | None = None
    speculative_draft_model_revision: str | None = None
    speculative_num_steps: int = 4
    speculative_eagle_topk: int = 5
    speculative_num_draft_tokens: int = 4
    speculative_accept_threshold_single: float = 1.0
    speculative_accept_threshold_acc: float = 1.0
    # --- sampling ----------------------------------------------------------------------------------
    enable_deterministic_sampling: bool = False
    enable_single_process: bool = False
    enable_nan_detection: bool = False
    use_sort_for_toppk_minp: bool = False
    # --- LoRA ------------------------------------------------------------------------------------------
    enable_lora: bool | None = None
    max_lora_rank: int | None = None
    lora_target_modules: list[str] | None = None
    lora_paths: list[str] | None = None
    max_loaded_loras: int | None = None
    max_loras_per_batch: int = 8
    lora_eviction_policy: str = field(default="lru", metadata=_m(choices=["lru", "fifo"]))
    enable_static_lora: bool | None = None
    lora_scaling: float | None = None
    enable_engine_loop_run_forever_daemon: bool | None = None
    multimodal: bool = False
    # --- expert balance / EPLB ------------------------------------------------------------------------------
    enable_return_routed_experts: bool = False
    enable_expert_balance_debug: bool = False
    expert_balance_segment_counter: int = 100
    expert_balance_output_file: str | None = None
    init_expert_location: str = "trivial"
    enable_expert_distribution_recorder: bool = False
    expert_distribution_recorder_buffer_size: int = 100
    expert_distribution_recorder_output_file: str | None = None
    # --- PD disaggregation (engine-level) -----------------------------------------------------------------------
    disaggregation_mode: str = field(default="null", metadata=_m(choices=["null", "prefill", "decode"]))
    disaggregation_bootstrap_url: str | None = None
    disaggregation_bootstrap_port: int = 8998
    disaggregation_transfer_port: int = 30001
    disaggregation_enable_d2h: bool = False
    # KV data path between engines of one NVLink domain: "cuda_ipc" lets the decode engine's page-copy kernel read
    # the prefill engine's pool directly; "tcp" stages through pinned host memory (works across nodes)
    disaggregation_transfer_backend: str = field(default="tcp", metadata=_m(choices=["tcp", "cuda_ipc"]))
    disaggregation_use_raiden: bool = False
    disaggregation_enable_chunk_prefill_transfer: bool = False
    disaggregation_side_channel_port: int = 9600
    disaggregation_d2h_pool_size: int = 64
    disaggregation_d2h_max_tokens: int | None = None
    disaggregation_channel_number: int = 4
    disaggregation_host_ip: str | None = None
    disaggregation_bootstrap_timeout_seconds: float = 5.0
    disaggregation_pull_timeout_seconds: float = 30.0
    disaggregation_ack_timeout_seconds: float = 60.0
    disaggregation_orphan_reaper_interval_seconds: float = 5.0
    disaggregation_shared_secret: str | None = None
    disaggregation_decode_watchdog_seconds: float = 0.0
    disaggregation_num_reserved_decode_tokens: int = 512
    disaggregation_max_inflight_transfers: int = 8
    # --- B200-specific (no counterpart in the reference) -----------------------------------------------------------
    disable_cuda_graph: bool = field(default=False, metadata=_m("run decode eagerly instead of replaying captured CUDA graphs"))
    cuda_graph_max_bs: int | None = field(default=None, metadata=_m("largest decode batch captured as a CUDA graph"))
    disable_fused_comm: bool = field(default=False, metadata=_m("use NCCL collectives instead of the fused GEMM+collective kernels"))
    disable_custom_kernels: bool = field(default=False, metadata=_m("run every op through its torch reference (CPU / debugging)"))

    # ------------------------------------------------------------------
    def __post_init__(self):
        if self.tokenizer_path is None:
            self.tokenizer_path = self.model_path
        if self.served_model_name is None:
            self.served_model_name = self.model_path
        if self.device is None:
            self.device = os.environ.get("SGLANG_DEVICE") or _default_device()
        if self.random_seed is None:
            self.random_seed = 42
        if self.mem_fraction_static is None:
            self.mem_fraction_static = 0.88
        if self.chunked_prefill_size is None:
            self.chunked_prefill_size = 4096
        if self.chunked_prefill_size is not None and self.chunked_prefill_size <= 0:
            self.chunked_prefill_size = -1  # disabled
        if self.grammar_backend is None:
            self.grammar_backend = "llguidance"
        if self.dp_schedule_policy is None:
            self.dp_schedule_policy = "round_robin" if self.disable_radix_cache else "cache_aware"
        if self.load_format == "random":
            self.load_format = "dummy"
        if self.attention_backend == "sm100":
            self.attention_backend = "fa"
        if self.device == "cpu":
            # No CUDA kernels, graphs or NCCL on a CPU-only host.
            self.disable_custom_kernels = True
            self.disable_cuda_graph = True
            self.disable_fused_comm = True
            self.attention_backend = "native"
        if self.enable_lora is None and self.lora_paths:
            self.enable_lora = True
        if self.max_loaded_loras is None and self.lora_paths:
            self.max_loaded_loras = max(len(self.lora_paths), self.max_loras_per_batch)
        if self.speculative_algorithm == "NEXTN":
            # MTP heads are loaded from the target checkpoint.
            if self.speculative_draft_model_path is None:
                self.speculative_draft_model_path = self.model_path
        if self.pd_disaggregation and self.disaggregation_mode == "null":
            # launcher-level flag: `disaggregation/local_pd.py` builds the prefill and decode engines from this one
            assert self.page_size >= 16, "PD mode requires a page_size of at least 16"
        self.check_server_args()

    # ------------------------------------------------------------------
    def check_server_args(self):
        """Cross-field validation (reference `server_args.py:1852-1932`)."""
        assert self.tp_size >= 1 and self.dp_size >= 1 and self.ep_size >= 1
        assert self.tp_size % self.nnodes == 0, "tp_size must be divisible by number of nodes"
        assert self.tp_size % self.dp_size == 0, "tp_size (total devices) must be divisible by dp_size"
        if self.chunked_prefill_size and self.chunked_prefill_size > 0:
            assert self.chunked_prefill_size % self.page_size == 0, (
                "chunked_prefill_size must be divisible by page_size")
        assert self.schedule_policy in SCHEDULE_POLICIES, f"unknown schedule_policy {self.schedule_policy}"
        assert self.dp_schedule_policy in DP_SCHEDULE_POLICIES
        assert 0.0 < self.mem_fraction_static < 1.0
        assert self.moe_backend in MOE_BACKENDS
        if self.speculative_algorithm is not None:
            assert self.speculative_algorithm in SPEC_ALGOS
            if self.speculative_algorithm == "DFLASH":
                assert self.speculative_draft_model_path, "DFLASH needs --speculative-draft-model-path"
            if self.speculative_algorithm in ("EAGLE", "EAGLE3", "STANDALONE"):
                assert self.speculative_draft_model_path, (
                    f"{self.speculative_algorithm} needs --speculative-draft-model-path")
            # Each speculative step needs the previous step's accepted tokens on the host.
            self.disable_overlap_schedule = True
            self.enable_mixed_chunk = False
        if self.disaggregation_mode != "null":
            if not self.disaggregation_bootstrap_url and os.environ.get("DISAGG_LAUNCH_BOOTSTRAP", "") == "1":
                # this engine hosts the registry itself, on --disaggregation-bootstrap-port
                host = self.disaggregation_host_ip or "127.0.0.1"
                self.disaggregation_bootstrap_url = f"http://{host}:{self.disaggregation_bootstrap_port}"
            assert self.disaggregation_bootstrap_url, "PD mode requires --disaggregation-bootstrap-url"
            assert self.page_size >= 16, "PD mode requires a page_size of at least 16"
        self.check_lora_server_args()

    def check_lora_server_args(self):
        """Reference `server_args.py:1934-2056`."""
        if not self.enable_lora:
            return
        assert self.max_loras_per_batch > 0
        if self.lora_paths is None:
            assert self.max_lora_rank and self.lora_target_modules, (
                "dynamic LoRA (no --lora-paths) requires --max-lora-rank and --lora-target-modules")
        if self.max_loaded_loras is not None:
            assert self.max_loaded_loras >= self.max_loras_per_batch

    # ------------------------------------------------------------------
    @staticmethod
    def add_cli_args(parser: argparse.ArgumentParser):
        for f in dataclasses.fields(ServerArgs):
            flag = "--" + f.name.replace("_", "-")
            names = [flag, *f.metadata.get("aliases", ())]
            kw: dict[str, Any] = {"dest": f.name, "help": f.metadata.get("help") or f.name.replace("_", " ")}
            tp, is_list, optional = _resolve_type(f.type)
            default = f.default if f.default is not dataclasses.MISSING else None
            if f.name == "model_path":
                names.append("--model")
                kw["required"] = True
            if tp is bool and not optional:
                kw["action"] = "store_true"
                kw["default"] = default
            elif tp is bool:
                kw["action"] = argparse.BooleanOptionalAction
                kw["default"] = default
            else:
                kw["type"] = tp
                kw["default"] = default
                if is_list:
                    kw["nargs"] = "+"
                ch = f.metadata.get("choices")
                if ch:
                    kw["choices"] = [c for c in ch if c is not None]
                if f.metadata.get("const") is not None:
                    kw["nargs"], kw["const"] = "?", f.metadata["const"]     # a bare flag takes this value
            parser.add_argument(*names, **kw)

    @classmethod
    def from_cli_args(cls, ns: argparse.Namespace) -> "ServerArgs":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in vars(ns).items() if k in names})

    @classmethod
    def from_cli(cls, argv: list[str] | None = None) -> "ServerArgs":
        parser = argparse.ArgumentParser(prog="sglang_jax_b200.launch_server")
        cls.add_cli_args(parser)
        return cls.from_cli_args(parser.parse_args(argv))

    def url(self) -> str:
        return f"http://{self.host}:{self.port}"

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    @property
    def tensor_size(self) -> int:
        """Width of the tensor axis: `tp_size` counts all devices, DP included."""
        return self.tp_size // self.dp_size


def _default_device() -> str:
    try:
        import torch
        return "cuda" if torch.cuda.is_available() else "cpu"
    except Exception:  # pragma: no cover
        return "cpu"


def _resolve_type(tp) -> tuple[type, bool, bool]:
    """Map a (string) annotation to (element type, is_list, is_optional)."""
    if isinstance(tp, str):
        tp = eval(tp, {"Any": Any})  # annotations are postponed in this module
    optional = False
    if get_origin(tp) is not None and type(None) in get_args(tp):
        optional = True
        tp = [a for a in get_args(tp) if a is not type(None)][0]
    if get_origin(tp) is list:
        return get_args(tp)[0], True, optional
    return tp, False, optional


def prepare_server_args(argv: list[str]) -> ServerArgs:
    return ServerArgs.from_cli(argv)


@dataclass
class PortArgs:
    """IPC endpoints of one engine (reference `server_args.py:2059-2097`)."""

    tokenizer_ipc_name: str
    scheduler_input_ipc_name: str
    detokenizer_ipc_name: str
    rpc_ipc_name: str
    metrics_ipc_name: str
    pub_sub_addr: str | None = None
    pub_sub_sync_addr: str | None = None
    nccl_port: int = 0

    @staticmethod
    def init_new(server_args: ServerArgs) -> "PortArgs":
        def ipc() -> str:
            f = tempfile.NamedTemporaryFile(prefix="sglb200_", delete=False)
            f.close()
            return f"ipc://{f.name}"

        pub = sync = None
        if server_args.nnodes > 1:
            host, port = (server_args.dist_init_addr or "127.0.0.1:25000").rsplit(":", 1)
            pub = f"tcp://{host}:{int(port) + 1}"
            sync = f"tcp://{host}:{int(port) + 2}"
        return PortArgs(ipc(), ipc(), ipc(), ipc(), ipc(), pub, sync,
                        nccl_port=random.randint(20000, 40000))


def parse_json_arg(s: str | None) -> dict:
    if not s:
        return {}
    return json.loads(s)
