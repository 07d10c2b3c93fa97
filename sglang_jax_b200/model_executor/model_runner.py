"""Per-GPU model executor.

Reference: `python/sgl_jax/srt/model_executor/model_runner.py:73-1106` plus the KV sizing
mixin (`model_runner_kv_cache_mixin.py`: cell size :293, `profile_max_num_token` :426,
`_resolve_max_num_reqs` :488, `init_memory_pool` :760).  Where the reference jit-compiles
one XLA executable per shape bucket, this runner launches hand-written kernels eagerly for
prefill and replays captured CUDA graphs for decode (`cuda_graph_runner.py`).
"""

from __future__ import annotations

import logging
import os
import time

import numpy as np
import torch

from .. import ops
from ..configs.model_config import AttentionArch, ModelConfig
from ..layers.radix_attention import AttentionBackend
from ..layers.sampler import Sampler, SamplingMetadata
from ..managers.schedule_batch import ForwardMode, ModelWorkerBatch
from ..mem_cache.memory_pool import MHATokenToKVPool, MLATokenToKVPool, ReqToTokenPool, SWAKVPool
from ..model_loader.loader import get_model_loader
from ..parallel import state as ps
from .forward_batch_info import ForwardBatch, _PinnedRing

logger = logging.getLogger(__name__)


def fused_token_window(server_args) -> tuple[int, int]:
    """`(min, max)` rows of the forwards that take the fused NVLink residual dataflow: empty by default,
    every forward with `--enable-sequence-parallel`; `SGLB_FUSED_MIN_TOKENS` / `SGLB_FUSED_MAX_TOKENS` override."""
    default_max = "1000000" if getattr(server_args, "enable_sequence_parallel", False) else "-1"
    return (int(os.environ.get("SGLB_FUSED_MIN_TOKENS", "0")), int(os.environ.get("SGLB_FUSED_MAX_TOKENS", default_max)))


class ModelRunner:
    def __init__(self, model_config: ModelConfig, server_args, device: str | torch.device | None = None,
                 req_to_token_pool: ReqToTokenPool | None = None, is_draft_worker: bool = False,
                 token_to_kv_pool=None, max_total_num_tokens: int | None = None):
        self.model_config = model_config
        self.server_args = server_args
        self.is_draft_worker = is_draft_worker
        st = ps.get_state()
        self.device = torch.device(device) if device is not None else st.device
        self.tp_size = st.tp.size
        self.tp_rank = st.tp.rank
        self.page_size = server_args.page_size
        self.dtype = model_config.dtype
        ops.set_force_reference(server_args.disable_custom_kernels or self.device.type == "cpu")
        self.attn_backend = AttentionBackend(
            "native" if (server_args.attention_backend == "native" or self.device.type == "cpu") else "fa")
        self.forward_ct = 0
        self.graph_replays = 0
        self.graph_recaptures = 0
        self.h2d_bytes_total = 0

        t0 = time.time()
        free_before = self._free_mem()
        loader = get_model_loader(server_args.load_format, seed=0)
        from ..configs.quantization_config import QuantizationConfig
        self.quant_config = QuantizationConfig.resolve(server_args.quantization, server_args.quantization_config_path,
                                                       model_config.hf_config)
        # expert placement (redundant experts, seeded from recorded load) and the hit-count recorder are fixed
        # before the routed-expert layers are built
        from ..layers.moe import configure_moe_runtime
        self.expert_recorder = None
        n_exp = int(getattr(model_config.hf_config, "num_experts", None)
                    or getattr(model_config.hf_config, "n_routed_experts", None)
                    or getattr(model_config.hf_config, "num_local_experts", None) or 0)
        if getattr(server_args, "enable_expert_balance_debug", False) and n_exp and not is_draft_worker:
            from ..eplb.expert_location import ExpertBalanceAnalyzer
            cfg = model_config.hf_text_config
            self.expert_recorder = ExpertBalanceAnalyzer(
                model_config.num_hidden_layers, n_exp + int(getattr(server_args, "ep_num_redundant_experts", 0) or 0),
                int(getattr(cfg, "num_experts_per_tok", None) or getattr(cfg, "top_k_experts", None) or 1),
                st.ep.size, server_args.expert_balance_segment_counter, server_args.expert_balance_output_file,
                device=self.device)
        elif getattr(server_args, "enable_expert_distribution_recorder", False) and n_exp and not is_draft_worker:
            from ..eplb.expert_location import ExpertDistributionRecorder
            self.expert_recorder = ExpertDistributionRecorder(
                model_config.num_hidden_layers, n_exp, server_args.expert_distribution_recorder_buffer_size,
                server_args.expert_distribution_recorder_output_file, device=self.device)
        configure_moe_runtime(getattr(server_args, "ep_num_redundant_experts", 0),
                              getattr(server_args, "init_expert_location", "trivial"), self.expert_recorder,
                              num_groups=getattr(model_config.hf_text_config, "n_group", 1) or 1,
                              num_nodes=getattr(server_args, "nnodes", 1) or 1,
                              dispatch_algorithm=getattr(server_args, "ep_dispatch_algorithm", None))
        self.model = loader.load_model(model_config, self.device, self.quant_config)
        configure_moe_runtime()          # later models (a draft head) start from the defaults
        from ..utils.debug_utils import print_parameter_shardings
        print_parameter_shardings(self.model)       # SGLANG_FRAMEWORK_LOG_LEVEL >= 3 only
        if not is_draft_worker:
            # `--moe-backend fused` / `fused_v2` / `auto`: token all-to-all between the expert-parallel ranks
            from ..layers import fused_ep_moe
            fused_ep_moe.ENABLED = server_args.moe_backend in ("fused", "fused_v2") or \
                (server_args.moe_backend == "auto" and st.ep.size > 1)
        self.weight_bytes = sum(p.numel() * p.element_size() for p in self.model.parameters())
        logger.info("model loaded in %.1fs, %.2f GB weights on %s", time.time() - t0,
                    self.weight_bytes / 2 ** 30, self.device)
        self.sampler = Sampler(server_args.random_seed, server_args.use_sort_for_toppk_minp,
                               server_args.enable_deterministic_sampling, server_args.enable_nan_detection)
        self._init_memory_pool(free_before, req_to_token_pool, token_to_kv_pool, max_total_num_tokens)
        self.staging = _PinnedRing(4, 1 << 16, str(self.device))
        # future-token map: slot = req row + 1; see `managers/tp_worker_overlap_thread.py`
        self.future_token_ids_map = torch.zeros(self.req_to_token_pool.size + 2, dtype=torch.int32,
                                                device=self.device)
        self.cuda_graph_runner = None
        self.lora_manager = None
        if server_args.enable_lora and not is_draft_worker:
            from ..lora.lora_manager import LoRAManager
            self.lora_manager = LoRAManager(self.model, server_args, self.dtype, self.device)
        self._init_fused_comm()
        self.routed_capturer = None
        if getattr(server_args, "enable_return_routed_experts", False) and not is_draft_worker:
            from ..layers.routed_experts_capturer import RoutedExpertsCapturer
            hf = model_config.hf_config
            cap_tokens = max(server_args.chunked_prefill_size or 0, server_args.max_prefill_tokens) + \
                self.max_running_requests
            self.routed_capturer = RoutedExpertsCapturer.attach(
                self.model, cap_tokens, self.device, int(getattr(hf, "num_experts_per_tok", None) or 8))
        from ..layers.fused_block import model_supports_fused_residual
        # the fused kernels read norm weights and row-parallel weights in the model dtype: per-module dtypes rule them out
        self.fused_residual_ok = model_supports_fused_residual(self.model) and \
            getattr(model_config, "dtype_config", None) is None
        # Forwards of `fused_min_tokens <= T <= fused_max_tokens` rows take the fused NVLink dataflow (one launch for
        # GEMM -> reduce-scatter -> residual + RMSNorm -> all-gather), the others GEMM + library all-reduce +
        # add-RMSNorm.  The default window is empty: measured end to end on Qwen3-32B with 128 running requests, the
        # library path is faster at two GPUs (decode step 15.6 ms against 17.5 ms, prefill steps equal) and at four
        # (17.4 ms against 19.3 ms per step).  The fused launch saves the reduction's latency but computes the
        # row-parallel product with its own small-M GEMM, which loses more than that against the measured per-shape
        # GEMM plan of the plain path.  `SGLB_FUSED_MAX_TOKENS=1000000` selects the fused dataflow for every forward,
        # `512` for decode-sized ones only.
        # `--enable-sequence-parallel` (reference `utils/parallel_utils.py`: reduce-scatter on the token dimension after a
        # row-parallel layer instead of an all-reduce) is this dataflow: it selects it for every forward
        self.fused_min_tokens, self.fused_max_tokens = fused_token_window(server_args)
        self.penalty_state = None          # sampling/penaltylib.PenaltyState, created when a request uses a penalty
        self.gemm_plan = None
        if self.device.type == "cuda" and os.environ.get("SGLB_GEMM_AUTOTUNE", "1") == "1" and not is_draft_worker:
            # measured GEMM plan, kept on disk between runs (counterpart of the reference's compile / AOT caches)
            from ..ops import native
            from .tuning_cache import GemmPlan
            self.gemm_plan = native.gemm_plan = GemmPlan(GemmPlan.default_path(native._LIB_PATH))
        if self.device.type == "cuda" and not server_args.disable_cuda_graph and not is_draft_worker:
            from .cuda_graph_runner import CudaGraphRunner
            self.cuda_graph_runner = CudaGraphRunner(self)
        if self.gemm_plan is not None:
            self.gemm_plan.save()

    # ------------------------------------------------------------------ memory
    def _free_mem(self) -> int:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            free, _ = torch.cuda.mem_get_info(self.device)
            return free
        import psutil
        return psutil.virtual_memory().available

    def _total_mem(self) -> int:
        if self.device.type == "cuda":
            return torch.cuda.mem_get_info(self.device)[1]
        import psutil
        return psutil.virtual_memory().total

    def cell_size(self) -> int:
        """Bytes of KV cache one token occupies on this rank."""
        mc = self.model_config
        kv_dtype = self.kv_cache_dtype
        n_layers = getattr(self.model, "num_kv_layers", None) or mc.num_hidden_layers
        if mc.attention_arch == AttentionArch.MLA:
            return MLATokenToKVPool.cell_size(mc.kv_lora_rank, mc.qk_rope_head_dim, n_layers, kv_dtype,
                                              getattr(self.model, "index_head_dim", 0))
        return MHATokenToKVPool.cell_size(mc.get_num_kv_heads(self.tp_size), mc.head_dim, n_layers, kv_dtype)

    def profile_max_num_token(self, free_before: int) -> int:
        if os.environ.get("SGLANG_CI_SMALL_KV_SIZE"):
            return int(os.environ["SGLANG_CI_SMALL_KV_SIZE"])
        total = self._total_mem()
        free_now = self._free_mem()
        if self.device.type == "cuda":
            rest = free_now - total * (1.0 - self.server_args.mem_fraction_static)
        else:
            rest = min(free_now * 0.25, 4 << 30)   # CPU runs are tests: stay small
        rest -= self._plan_recurrent_pool(rest)
        n = int(rest // self.cell_size())
        if self.tp_size > 1:
            t = torch.tensor([n], dtype=torch.int64)
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=ps.get_state().tp.cpu_group)
            n = int(t.item())
        return n

    def _plan_recurrent_pool(self, available_bytes: float) -> int:
        """Hybrid linear-attention models: decide the number of checkpoint slots of the recurrent state pool from
        `--max-recurrent-state-size` / `--recurrent-snapshot-slots` / `--recurrent-state-memory-ratio` and return the
        bytes the pool will take, which come out of the KV budget."""
        spec = getattr(self.model, "recurrent_spec", None)
        if not spec:
            return 0
        from ..mem_cache.recurrent_state_pool import plan_state_slots, slot_bytes
        sa = self.server_args
        reqs = (sa.max_running_requests or 256) + 8
        per = slot_bytes(conv_dtype=self.dtype, **spec)
        self._recurrent_snapshots, used = plan_state_slots(
            reqs, per, int(max(available_bytes, 0)), sa.max_recurrent_state_size, int(sa.recurrent_snapshot_slots),
            float(sa.recurrent_state_memory_ratio), not sa.disable_radix_cache)
        logger.info("recurrent state pool: %d request + %d checkpoint slots of %.2f MB", reqs,
                    self._recurrent_snapshots, per / 2 ** 20)
        return used

    def _init_memory_pool(self, free_before, req_to_token_pool, token_to_kv_pool, max_total):
        sa, mc = self.server_args, self.model_config
        kvd = sa.kv_cache_dtype
        self.kv_cache_dtype = {"auto": self.dtype, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
                               "fp8_e4m3": torch.float8_e4m3fn, "fp8_e5m2": torch.float8_e5m2}[kvd]
        if token_to_kv_pool is not None:
            # draft worker shares the target's row table and allocator; it owns its own KV tensors
            self.max_total_num_tokens = max_total
        else:
            n = self.profile_max_num_token(free_before)
            if sa.max_total_tokens is not None:
                n = min(n, sa.max_total_tokens)
            n = n // self.page_size * self.page_size
            if n <= 0:
                raise RuntimeError("Not enough memory for the KV cache; raise --mem-fraction-static")
            self.max_total_num_tokens = n
        ctx = mc.context_len
        max_reqs = sa.max_running_requests
        if max_reqs is None:
            max_reqs = min(max(int(self.max_total_num_tokens / ctx * 512), 256), 2048)
        self.max_running_requests = max_reqs
        if req_to_token_pool is None:
            # a few spare rows: requests being chunk-prefilled or retracted hold rows too
            req_to_token_pool = ReqToTokenPool(max_reqs + 8, ctx + 8, str(self.device), self.page_size)
        self.req_to_token_pool = req_to_token_pool
        self.recurrent_pool = None
        spec = getattr(self.model, "recurrent_spec", None)
        if spec:
            from ..mem_cache.recurrent_state_pool import RecurrentStatePool
            # one state slot per request row (slot = row + 1)
            snap = getattr(self, "_recurrent_snapshots", None)
            if snap is None:         # the KV size was given from outside (draft worker, CI size): plan without a budget
                from ..mem_cache.recurrent_state_pool import plan_state_slots, slot_bytes
                snap, _ = plan_state_slots(req_to_token_pool.size, slot_bytes(conv_dtype=self.dtype, **spec), 0,
                                           sa.max_recurrent_state_size, max(int(sa.recurrent_snapshot_slots), 0),
                                           float(sa.recurrent_state_memory_ratio), not sa.disable_radix_cache)
            self.recurrent_pool = RecurrentStatePool(req_to_token_pool.size, device=str(self.device),
                                                     conv_dtype=self.dtype, snapshot_slots=snap, **spec)
        n_layers = getattr(self.model, "num_kv_layers", None) or mc.num_hidden_layers
        if mc.attention_arch == AttentionArch.MLA:
            self.token_to_kv_pool = MLATokenToKVPool(self.max_total_num_tokens, self.page_size, self.kv_cache_dtype,
                                                     mc.kv_lora_rank, mc.qk_rope_head_dim, n_layers, str(self.device),
                                                     index_head_dim=getattr(self.model, "index_head_dim", 0))
        elif getattr(self.model, "swa_layer_ids", None) and (not sa.disable_hybrid_swa_memory
                                                            or hasattr(self.model, "swa_kv_shape")):
            swa_ids = self.model.swa_layer_ids
            full_ids = [i for i in range(mc.num_hidden_layers) if i not in set(swa_ids)]
            ratio = sa.swa_full_tokens_ratio
            full = self.max_total_num_tokens
            swa = max(int(full * ratio) // self.page_size * self.page_size, self.page_size)
            fh, fd = getattr(self.model, "full_kv_shape", None) or (mc.get_num_kv_heads(self.tp_size), mc.head_dim)
            self.token_to_kv_pool = SWAKVPool(full, swa, self.page_size, self.kv_cache_dtype, fh, fd, swa_ids, full_ids,
                                              str(self.device), *getattr(self.model, "swa_kv_shape", ()))
        else:
            heads, dim = getattr(self.model, "kv_shape", None) or (mc.get_num_kv_heads(self.tp_size), mc.head_dim)
            self.token_to_kv_pool = MHATokenToKVPool(self.max_total_num_tokens, self.page_size, self.kv_cache_dtype,
                                                     heads, dim, n_layers, str(self.device))
        logger.info("KV pool: %d tokens, %.2f GB, max_running_requests=%d", self.max_total_num_tokens,
                    self.token_to_kv_pool.get_kv_size_bytes() / 2 ** 30, max_reqs)
        if self.device.type == "cuda" and os.environ.get("SGLB_BOUNDS_CHECK", "0") == "1":
            # checked build of the kernel library: the KV-write kernel verifies its slots against the pool's extent
            from ..ops import native
            pages = max(p.num_pages for p in (getattr(self.token_to_kv_pool, "full_pool", self.token_to_kv_pool),
                                              getattr(self.token_to_kv_pool, "swa_pool", self.token_to_kv_pool)))
            if native.set_debug_kv_pages(pages):
                logger.info("checked kernel build: KV writes are verified against %d pages", pages)

    def _init_fused_comm(self):
        st = ps.get_state()
        want = (self.tp_size > 1 and self.device.type == "cuda" and not self.server_args.disable_fused_comm
                and not self.server_args.disable_custom_kernels and st.fused_comm is None)
        if not want:
            return
        ok = 1
        try:
            from ..parallel.fused_comm import FusedComm
            sa = self.server_args
            max_tokens = max(sa.chunked_prefill_size or 0, sa.max_prefill_tokens) + self.max_running_requests
            st.fused_comm = FusedComm.create(st, self.model_config.hidden_size, self.dtype, max_tokens)
        except Exception as e:  # NCCL path remains fully functional
            logger.warning("fused communication kernels unavailable (%s); using NCCL", e)
            ok = 0
        # all ranks must take the same path
        import torch.distributed as dist
        t = torch.tensor([ok], dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=st.tp.cpu_group)
        if int(t.item()) == 0:
            st.fused_comm = None

    # ------------------------------------------------------------------ forward
    def select_residual_dataflow(self, fb) -> bool:
        """Choose, once per model forward, between the token-sharded residual stream of the fused NVLink kernels
        and the replicated one of the library all-reduce.  Anything that reads whole rows of the residual between
        layers (deep-stack features, auxiliary hidden-state capture for EAGLE-3 / DFlash, the precision tracer) or
        a layer that cannot feed the fused reduce (LoRA on a row-parallel projection) selects the replicated one
        for the whole forward."""
        from ..layers.fused_block import set_fused_residual
        from ..utils.precision_tracer import precision_tracer
        inner = getattr(self.model, "model", None)
        on = (self.fused_residual_ok and not precision_tracer.enabled
              and (fb is None or self.fused_min_tokens <= fb.num_tokens <= self.fused_max_tokens)
              and (fb is None or fb.extras.get("deepstack") is None)
              and not getattr(inner, "layers_to_capture", None)
              and not getattr(self.model, "capture_aux_hidden_states", False))
        set_fused_residual(on)
        return on

    def resolve_future_token_ids(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Negative ids are placeholders `-slot` for tokens the previous step is still
        sampling; replace them from the device-side future map."""
        return torch.where(input_ids < 0, self.future_token_ids_map[(-input_ids).clamp_min(0).long()], input_ids)

    @torch.inference_mode()
    def forward(self, batch: ModelWorkerBatch, skip_sample: bool = False):
        """One step: returns `(logits_output, next_token_ids [B] int32 device tensor, forward_batch)`."""
        self.forward_ct += 1
        if self.expert_recorder is not None:
            if hasattr(self.expert_recorder, "flush_segment"):      # balance debug counts decode steps only
                self.expert_recorder.step(batch.forward_mode.is_decode())
            else:
                self.expert_recorder.step()
        if batch.forward_mode.is_idle():
            return None, torch.empty(0, dtype=torch.int32, device=self.device), None
        if getattr(batch, "recurrent_copies", None) and self.recurrent_pool is not None:
            self.recurrent_pool.copy_sequence(batch.recurrent_copies)      # prefix-cache checkpoints / clones
        gr = self.cuda_graph_runner
        if gr is not None and gr.can_run(batch):
            return gr.replay(batch)
        fb = ForwardBatch.init_new(batch, self)
        self.h2d_bytes_total += fb.h2d_bytes
        si = batch.spec_info
        if si is not None:
            # speculative forwards keep their token ids / positions on the device
            if getattr(si, "input_ids", None) is not None:
                fb.input_ids = si.input_ids
            if getattr(si, "positions", None) is not None:
                fb.positions = si.positions
            if getattr(si, "all_logits", False):
                fb.last_token_indices = None
        if self.server_args is not None and not self.server_args.disable_overlap_schedule:
            fb.input_ids = self.resolve_future_token_ids(fb.input_ids)
        comm = ps.get_state().fused_comm
        self.select_residual_dataflow(fb)
        si = batch.sampling_info
        if (comm is not None and not skip_sample and not batch.return_logprob and si is not None and si.is_all_greedy
                and si.linear_penalty is None and si.vocab_mask is None and si.logit_bias is None
                and getattr(si, "penalties", None) is None
                and batch.capture_hidden_mode == 0 and len(batch.req_pool_indices) <= 1024):
            fb.extras["skip_logits_gather"] = True     # greedy: reduce (max, index) pairs, not logits
        if self.lora_manager is not None:
            from ..lora.context_manager import lora_batch
            per_req = batch.extend_seq_lens if batch.forward_mode.is_extend() else np.ones(len(batch.req_pool_indices), np.int64)
            with lora_batch(self.lora_manager.prepare_batch(batch.lora_ids, per_req)):
                out = self.model(fb.input_ids, fb)
        elif getattr(batch, "input_embeds", None) is not None:
            emb = batch.input_embeds.to(self.device, self.dtype)
            if getattr(batch, "input_embeds_rows", None) is not None and not batch.input_embeds_rows.all():
                # rows without encoder embeddings (other requests of the batch) use the token table
                embed = getattr(self.model, "embed_input_ids", None) or self.model.model.embed_tokens
                rows = torch.from_numpy(batch.input_embeds_rows).to(self.device)
                emb = torch.where(rows[:, None], emb, embed(fb.input_ids).to(emb.dtype))
            out = self.model(fb.input_ids, fb, emb)
        else:
            out = self.model(fb.input_ids, fb)
        if skip_sample:
            return out, None, fb
        if "vocab_shard" in out.extras:
            start, vocab = out.extras["vocab_shard"]
            ids = comm.argmax_gather(out.next_token_logits, start, vocab)
        else:
            if si is not None and getattr(si, "penalties", None) is not None:
                # frequency / presence penalties, min_new_tokens: token counts per request slot live on the device
                # and are brought up to date from this step's (resolved) input ids
                if self.penalty_state is None:
                    from ..sampling.penaltylib import PenaltyState
                    self.penalty_state = PenaltyState(self.req_to_token_pool.size + 1, out.next_token_logits.shape[-1],
                                                      self.device)
                decode = batch.forward_mode.is_decode()
                out.next_token_logits = self.penalty_state.apply(out.next_token_logits, si.penalties,
                                                                 batch.req_pool_indices,
                                                                 fb.input_ids if decode else None, decode)
            meta = SamplingMetadata.from_worker_batch(batch, self.device)
            ids = self.sampler(out, meta)
        if batch.future_slots is not None:
            slots = torch.from_numpy(batch.future_slots).to(self.device, non_blocking=True).long()
            self.future_token_ids_map[slots] = ids
        return out, ids, fb

    def sample(self, logits_output, batch: ModelWorkerBatch):
        return self.sampler(logits_output, SamplingMetadata.from_worker_batch(batch, self.device))
