"""Request and batch state of the scheduler.

`Req` is one generation request; `ScheduleBatch` is the scheduler's mutable view
of the requests that run together; `ModelWorkerBatch` is the immutable snapshot
handed (and, under tensor parallelism, broadcast) to the model workers.

Semantics follow the reference's `python/sgl_jax/srt/managers/schedule_batch.py`
(finish reasons :95-164, `Req` :167-703, `ScheduleBatch` :837-3500,
`ModelWorkerBatch` :3648).  Differences that come from the B200 design:

* batches are not padded to shape buckets on the host — CUDA-graph replay pads
  on the device side, so the snapshot carries exact sizes;
* the snapshot carries *page-table deltas* (request row, page position, page id)
  instead of a rebuilt page list, because workers keep a persistent device page
  table (see `mem_cache/memory_pool.py`).
"""

from __future__ import annotations

import dataclasses
import logging
import time
from enum import IntEnum
from typing import Any

import numpy as np

from ..global_config import global_config
from ..mem_cache.radix_cache import RadixKey
from ..sampling.sampling_params import SamplingParams

logger = logging.getLogger(__name__)

INIT_INCREMENTAL_DETOKENIZATION_OFFSET = 5


# --------------------------------------------------------------------------- finish reasons
class BaseFinishReason:
    def __init__(self, is_error: bool = False):
        self.is_error = is_error

    def to_json(self) -> dict:
        raise NotImplementedError


class FINISH_MATCHED_TOKEN(BaseFinishReason):
    def __init__(self, matched: int | list[int]):
        super().__init__()
        self.matched = matched

    def to_json(self):
        return {"type": "stop", "matched": self.matched}


class FINISH_MATCHED_STR(BaseFinishReason):
    def __init__(self, matched: str):
        super().__init__()
        self.matched = matched

    def to_json(self):
        return {"type": "stop", "matched": self.matched}


class FINISH_LENGTH(BaseFinishReason):
    def __init__(self, length: int):
        super().__init__()
        self.length = length

    def to_json(self):
        return {"type": "length", "length": self.length}


class FINISH_ABORT(BaseFinishReason):
    def __init__(self, message: str = "Aborted", status_code: int | None = None, err_type: str | None = None):
        super().__init__(is_error=True)
        self.message = message
        self.status_code = status_code
        self.err_type = err_type

    def to_json(self):
        return {"type": "abort", "message": self.message, "status_code": self.status_code,
                "err_type": self.err_type}


# --------------------------------------------------------------------------- forward mode
class ForwardMode(IntEnum):
    EXTEND = 1
    DECODE = 2
    MIXED = 3
    IDLE = 4
    TARGET_VERIFY = 5
    DRAFT_EXTEND = 6
    DUMMY_FIRST = 7

    def is_extend(self):
        return self in (ForwardMode.EXTEND, ForwardMode.MIXED, ForwardMode.DRAFT_EXTEND,
                        ForwardMode.TARGET_VERIFY)

    def is_decode(self):
        return self == ForwardMode.DECODE

    def is_mixed(self):
        return self == ForwardMode.MIXED

    def is_idle(self):
        return self == ForwardMode.IDLE

    def is_target_verify(self):
        return self == ForwardMode.TARGET_VERIFY

    def is_draft_extend(self):
        return self == ForwardMode.DRAFT_EXTEND

    def is_decode_or_idle(self):
        return self in (ForwardMode.DECODE, ForwardMode.IDLE)


# --------------------------------------------------------------------------- request
class Req:
    def __init__(self, rid: str, origin_input_text: str | None, origin_input_ids: list[int],
                 sampling_params: SamplingParams, return_logprob: bool = False,
                 top_logprobs_num: int = 0, token_ids_logprob: list[int] | None = None,
                 stream: bool = False, origin_input_ids_unpadded=None, lora_id: str | None = None,
                 eos_token_ids: set[int] | None = None, vocab_size: int | None = None,
                 extra_key: str | None = None, dp_rank: int | None = None,
                 return_hidden_states: bool = False, return_routed_experts: bool = False,
                 return_output_logprob_only: bool = False, logprob_start_len: int = -1,
                 session_id: str | None = None, bootstrap_host=None, bootstrap_port=None,
                 bootstrap_room=None, mm_inputs: dict | None = None):
        self.rid = rid
        # encoder-stage products: "input_embedding" [prompt_len, hidden], "mrope_positions"
        # [3, prompt_len], "mrope_position_delta" (3-D position minus token index after the prompt)
        self.mm_inputs = mm_inputs
        self.origin_input_text = origin_input_text
        self.origin_input_ids = list(origin_input_ids)
        self.origin_input_ids_unpadded = origin_input_ids_unpadded or self.origin_input_ids
        self.output_ids: list[int] = []
        self.fill_ids: list[int] = []
        self.sampling_params = sampling_params
        self.lora_id = lora_id
        self.extra_key = extra_key
        self.dp_rank = dp_rank
        self.session_id = session_id
        self.vocab_size = vocab_size
        self.eos_token_ids = eos_token_ids
        self.tokenizer = None

        # memory
        self.req_pool_idx: int | None = None
        self.prefix_indices: np.ndarray = np.empty(0, np.int32)
        self.last_matched_prefix_len = 0
        self.extend_input_len = 0
        self.last_node: Any = None
        self.last_host_node: Any = None
        self.host_token_pending = False     # latest token known on the host only (arrived with transferred KV)
        self.penalty_restart = False        # this step must (re)build the request's device-side token counts
        self.swa_evicted_seqlen = 0          # SWA slots before this position were already released
        self.host_hit_length = 0
        self.cached_tokens = 0
        self.already_computed = 0
        self.is_chunked = 0
        self.is_retracted = False
        self.kv_committed_len = 0   # tokens whose KV is written
        self.kv_allocated_len = 0   # slots recorded in the request's row

        # finish state
        self.finished_reason: BaseFinishReason | None = None
        self.finished_len: int | None = None
        self.to_abort = False
        self.to_abort_message = ""
        self.stream = stream

        # incremental detokenisation
        self.decoded_text = ""
        self.surr_offset: int | None = None
        self.read_offset: int | None = None
        self.send_token_offset = 0
        self.send_decode_id_offset = 0
        self.send_output_token_logprobs_offset = 0

        # logprobs
        self.return_logprob = return_logprob
        self.return_output_logprob_only = return_output_logprob_only
        self.logprob_start_len = logprob_start_len
        self.top_logprobs_num = top_logprobs_num
        self.token_ids_logprob = token_ids_logprob
        self.extend_logprob_start_len = 0
        self.input_token_logprobs_val: list | None = None
        self.input_token_logprobs_idx: list | None = None
        self.input_top_logprobs_val: list | None = None
        self.input_top_logprobs_idx: list | None = None
        self.input_token_ids_logprobs_val: list | None = None
        self.input_token_ids_logprobs_idx: list | None = None
        self.input_logprob_sent = False
        self.output_token_logprobs_val: list = []
        self.output_token_logprobs_idx: list = []
        self.output_top_logprobs_val: list = []
        self.output_top_logprobs_idx: list = []
        self.output_token_ids_logprobs_val: list = []
        self.output_token_ids_logprobs_idx: list = []
        self.return_hidden_states = return_hidden_states
        self.hidden_states: list = []
        self.return_routed_experts = return_routed_experts
        self.routed_experts: list = []

        # grammar
        self.grammar: Any = None
        self.grammar_key: tuple | None = None
        self.grammar_wait_ct = 0

        # speculative decoding
        self.spec_verify_ct = 0
        self.spec_accepted_tokens = 0

        # PD disaggregation
        self.bootstrap_host = bootstrap_host
        self.bootstrap_port = bootstrap_port
        self.bootstrap_room = bootstrap_room
        self.disagg_kv_sender = None
        self.disagg_kv_receiver = None

        # timing
        self.queue_time_start = time.perf_counter()
        self.queue_time_end: float | None = None
        self.first_token_time: float | None = None
        self.finished_time: float | None = None

    # ---------------------------------------------------------------------
    @property
    def seqlen(self) -> int:
        return len(self.origin_input_ids) + len(self.output_ids)

    def finished(self) -> bool:
        return self.finished_reason is not None

    def committed_kv_len(self) -> int:
        """Tokens whose KV is in the pool: everything but the last sampled token,
        which is only written when it is fed to the next step."""
        return self.kv_committed_len

    def init_next_round_input(self, tree_cache=None):
        """Compute `fill_ids` and match the longest cached prefix (reference
        `schedule_batch.py:433-525`): at least one token is always recomputed so the
        step produces logits."""
        self.fill_ids = self.origin_input_ids + self.output_ids
        input_len = len(self.fill_ids)
        max_prefix_len = input_len - 1
        if self.return_logprob and not self.return_output_logprob_only and self.logprob_start_len >= 0:
            max_prefix_len = min(max_prefix_len, self.logprob_start_len)
        max_prefix_len = max(max_prefix_len, 0)
        if tree_cache is not None:
            res = tree_cache.match_prefix(
                RadixKey(self.fill_ids[:max_prefix_len], self.extra_key, self.dp_rank or 0), req=self)
            self.prefix_indices = res.device_indices
            self.last_node = res.last_device_node
            self.last_host_node = res.last_host_node
            self.host_hit_length = res.host_hit_length
            self.last_matched_prefix_len = len(self.prefix_indices)
        self.extend_input_len = len(self.fill_ids) - len(self.prefix_indices)

    def adjust_max_prefix_ids(self):
        return self.fill_ids[: max(len(self.fill_ids) - 1, 0)]

    def init_incremental_detokenize(self):
        first_iter = self.surr_offset is None or self.read_offset is None
        if first_iter:
            self.read_offset = len(self.origin_input_ids_unpadded)
            self.surr_offset = max(self.read_offset - INIT_INCREMENTAL_DETOKENIZATION_OFFSET, 0)
        all_ids = self.origin_input_ids_unpadded + self.output_ids
        return all_ids[self.surr_offset:], self.read_offset - self.surr_offset

    def check_finished(self, new_accepted_len: int = 1):
        """Reference `schedule_batch.py:573-654`."""
        if self.finished():
            return
        if self.to_abort:
            self.finished_reason = FINISH_ABORT(self.to_abort_message or "Aborted")
            return
        sp = self.sampling_params
        if len(self.output_ids) >= sp.max_new_tokens:
            self.finished_reason = FINISH_LENGTH(length=sp.max_new_tokens)
            self.finished_len = sp.max_new_tokens
            return
        if self.grammar is not None and getattr(self.grammar, "is_terminated", lambda: False)():
            self.finished_reason = FINISH_MATCHED_TOKEN(matched=self.output_ids[-1])
            return
        new_tokens = self.output_ids[-new_accepted_len:]
        if not sp.ignore_eos:
            for j, tok in enumerate(new_tokens):
                matched = False
                if sp.stop_token_ids and tok in sp.stop_token_ids:
                    matched = True
                elif self.eos_token_ids and tok in self.eos_token_ids:
                    matched = True
                elif self.tokenizer is not None and getattr(self.tokenizer, "eos_token_id", None) == tok:
                    matched = True
                elif self.tokenizer is not None and tok in (getattr(self.tokenizer, "additional_stop_token_ids", None) or ()):
                    matched = True
                if matched:
                    self.finished_reason = FINISH_MATCHED_TOKEN(matched=tok)
                    self.finished_len = len(self.output_ids) - len(new_tokens) + j + 1
                    return
        if self.vocab_size is not None:
            for tok in new_tokens:
                if tok > self.vocab_size or tok < 0:
                    # garbage from a NaN forward: stop instead of feeding it back
                    self.output_ids[-1] = next(iter(self.eos_token_ids)) if self.eos_token_ids else 0
                    self.finished_reason = FINISH_MATCHED_STR(matched="NaN happened")
                    return
        if sp.stop_strs and self.tokenizer is not None:
            tail = self.tokenizer.decode(self.output_ids[-(sp.stop_str_max_len + 1):])
            for s in sp.stop_strs:
                if s in tail or s in self.decoded_text:
                    self.finished_reason = FINISH_MATCHED_STR(matched=s)
                    return

    def reset_for_retract(self):
        """Return to the just-arrived state, keeping generated tokens: the request will
        be re-prefilled over prompt + output (reference :656-703)."""
        self.prefix_indices = np.empty(0, np.int32)
        self.last_matched_prefix_len = 0
        self.last_node = None
        self.extend_input_len = 0
        self.is_retracted = True
        self.is_chunked = 0
        self.req_pool_idx = None
        self.already_computed = 0
        self.kv_committed_len = 0
        self.kv_allocated_len = 0
        self.swa_evicted_seqlen = 0
        self.routed_experts = []       # the re-prefill computes (and records) every token again
        self.input_token_logprobs_val = None if not self.input_logprob_sent else self.input_token_logprobs_val

    def offload_kv_cache(self, *a, **k):  # hook used by HiCache / PD
        pass

    def __repr__(self):
        return (f"Req(rid={self.rid}, in={len(self.origin_input_ids)}, out={len(self.output_ids)}, "
                f"prefix={len(self.prefix_indices)}, chunked={self.is_chunked})")


# --------------------------------------------------------------------------- sampling snapshot
@dataclasses.dataclass
class ModelWorkerSamplingInfo:
    """Per-row sampling controls of one batch (reference `schedule_batch.py:3507`)."""

    temperatures: np.ndarray          # f32 [bs]
    top_ps: np.ndarray                # f32 [bs]
    top_ks: np.ndarray                # i32 [bs]
    min_ps: np.ndarray                # f32 [bs]
    sampling_seeds: np.ndarray | None  # i32 [bs] or None
    is_all_greedy: bool
    need_top_p_sampling: bool
    need_top_k_sampling: bool
    need_min_p_sampling: bool
    linear_penalty: np.ndarray | None = None   # f32 [bs, vocab] additive
    vocab_mask: np.ndarray | None = None       # i32 [bs, ceil(vocab/32)], bit set = allowed
    logit_bias: np.ndarray | None = None
    positions: np.ndarray | None = None        # i32 [bs]: position of the token being sampled
    penalties: object | None = None            # `sampling.penaltylib.PenaltyInfo` when a request uses a penalty

    @staticmethod
    def from_reqs(reqs: list[Req], vocab_size: int, penalizer=None) -> "ModelWorkerSamplingInfo":
        n = len(reqs)
        t = np.empty(n, np.float32)
        p = np.empty(n, np.float32)
        k = np.empty(n, np.int32)
        m = np.empty(n, np.float32)
        seeds = None
        for i, r in enumerate(reqs):
            sp = r.sampling_params
            t[i] = sp.temperature
            p[i] = sp.top_p
            k[i] = min(sp.top_k, vocab_size)
            m[i] = sp.min_p
            if sp.sampling_seed is not None:
                if seeds is None:
                    seeds = np.full(n, 42, np.int32)
                seeds[i] = np.int32(np.uint32(sp.sampling_seed & 0xFFFFFFFF))
        bias = None
        for i, r in enumerate(reqs):
            lb = r.sampling_params.logit_bias
            if lb:
                if bias is None:
                    bias = np.zeros((n, vocab_size), np.float32)
                for tok, v in lb.items():
                    bias[i, int(tok)] = v
        return ModelWorkerSamplingInfo(
            temperatures=t, top_ps=p, top_ks=k, min_ps=m, sampling_seeds=seeds,
            is_all_greedy=bool((k <= 1).all()),
            need_top_p_sampling=bool((p < 1.0).any()),
            need_top_k_sampling=bool((k < vocab_size).any()),
            need_min_p_sampling=bool((m > 0).any()),
            logit_bias=bias,
            positions=np.array([r.seqlen for r in reqs], np.int32),
        )


# --------------------------------------------------------------------------- worker batch
@dataclasses.dataclass
class ModelWorkerBatch:
    bid: int
    forward_mode: ForwardMode
    input_ids: np.ndarray            # i32 [T]; negative = future-token placeholder
    req_pool_indices: np.ndarray     # i32 [B]
    seq_lens: np.ndarray             # i32 [B] KV length after this step
    out_cache_loc: np.ndarray        # i32 [T]
    positions: np.ndarray            # i32 [T]
    extend_prefix_lens: np.ndarray | None = None   # i32 [B]
    extend_seq_lens: np.ndarray | None = None      # i32 [B]
    extend_logprob_start_lens: np.ndarray | None = None
    page_delta_rows: np.ndarray | None = None      # i32 [N] request rows
    page_delta_pos: np.ndarray | None = None       # i32 [N] page positions
    page_delta_ids: np.ndarray | None = None       # i32 [N] page ids
    sampling_info: ModelWorkerSamplingInfo | None = None
    return_logprob: bool = False
    top_logprobs_nums: list[int] | None = None
    token_ids_logprobs: list | None = None
    return_output_logprob_only: bool = False
    capture_hidden_mode: int = 0
    return_routed_experts: bool = False      # some request of the batch wants its routed expert ids back
    lora_ids: list | None = None
    num_decode_in_mixed: int = 0     # MIXED: trailing rows that are 1-token decodes
    spec_info: Any = None
    spec_algorithm: Any = None
    dp_rank: int = 0
    real_bs: int = 0
    launch_done: Any = None
    # ids of future-map slots the sampled tokens must be stored to (overlap mode)
    future_slots: np.ndarray | None = None
    # [T, hidden] embeddings that replace the token embedding lookup (multimodal prefill);
    # with `input_embeds_rows` (bool [T]) only the marked rows are replaced
    input_embeds: Any = None
    input_embeds_rows: np.ndarray | None = None
    # i32 [3, T] (temporal, height, width) positions for multimodal rotary embeddings
    mrope_positions: np.ndarray | None = None
    # [L, T, hidden]: vision features added to the residual stream after each of the first L layers
    deepstack_embeds: Any = None
    # (src, dst) recurrent-state slot copies to run, in order, before this forward
    recurrent_copies: list | None = None
    # (index of the sequence in the batch, tokens of this extend before the checkpoint, snapshot slot): the
    # linear-attention layers store their state after that many tokens of the sequence into the slot
    recurrent_tracks: list | None = None

    @property
    def batch_size(self):
        return len(self.req_pool_indices)

    @property
    def num_tokens(self):
        return len(self.input_ids)


# --------------------------------------------------------------------------- schedule batch
_bid = 0


def _next_bid() -> int:
    global _bid
    _bid += 1
    return _bid


class ScheduleBatch:
    def __init__(self, reqs: list[Req], req_to_token_pool, token_to_kv_pool_allocator, tree_cache,
                 vocab_size: int, enable_overlap: bool = False, page_size: int = 1,
                 spec_algorithm=None, dp_rank: int = 0):
        self.reqs = reqs
        self.req_to_token_pool = req_to_token_pool
        self.token_to_kv_pool_allocator = token_to_kv_pool_allocator
        self.tree_cache = tree_cache
        self.vocab_size = vocab_size
        self.enable_overlap = enable_overlap
        self.page_size = page_size
        self.spec_algorithm = spec_algorithm
        self.dp_rank = dp_rank
        self.forward_mode: ForwardMode | None = None
        self.batch_is_full = False
        self.chunked_req: Req | None = None
        self.decoding_reqs: list[Req] | None = None   # mixed-chunk: decode rows merged in
        self.num_decode_in_mixed = 0

        self.input_ids: np.ndarray | None = None
        self.output_ids: np.ndarray | None = None     # last sampled ids (may be placeholders)
        self.req_pool_indices: np.ndarray | None = None
        self.seq_lens: np.ndarray | None = None
        self.out_cache_loc: np.ndarray | None = None
        self.prefix_lens: list[int] = []
        self.extend_lens: list[int] = []
        self.extend_num_tokens = 0
        self.extend_logprob_start_lens: list[int] = []
        self.return_logprob = any(r.return_logprob for r in reqs)
        self.return_hidden_states = any(r.return_hidden_states for r in reqs)
        self.has_stream = any(r.stream for r in reqs)
        self.has_grammar = any(r.grammar is not None for r in reqs)
        self.spec_info = None

    @classmethod
    def init_new(cls, reqs, req_to_token_pool, token_to_kv_pool_allocator, tree_cache, vocab_size,
                 enable_overlap=False, page_size=1, spec_algorithm=None, chunked_req=None, dp_rank=0):
        b = cls(reqs, req_to_token_pool, token_to_kv_pool_allocator, tree_cache, vocab_size,
                enable_overlap, page_size, spec_algorithm, dp_rank)
        b.chunked_req = chunked_req
        return b

    def batch_size(self) -> int:
        return len(self.reqs)

    def is_empty(self) -> bool:
        return len(self.reqs) == 0

    # ------------------------------------------------------------------ memory helpers
    def _evict_then(self, need_tokens: int, fn):
        alloc = self.token_to_kv_pool_allocator
        out = fn()
        if out is None and self.tree_cache is not None:
            self._cache_evict(need_tokens)
            out = fn()
        return out

    def _cache_evict(self, need_tokens: int):
        if hasattr(self.tree_cache, "swa_evictable_size"):
            self.tree_cache.evict(need_tokens, need_tokens)      # (full, sliding-window) budgets
        else:
            self.tree_cache.evict(need_tokens, dp_rank=self.dp_rank)

    # ------------------------------------------------------------------ extend
    def prepare_for_extend(self):
        """Allocate request rows and KV slots for a prefill step and lay out the
        flattened token arrays (reference `schedule_batch.py:1177-1411`)."""
        self.forward_mode = ForwardMode.EXTEND
        reqs = self.reqs
        pool = self.req_to_token_pool
        need_rows = sum(1 for r in reqs if r.req_pool_idx is None)
        rows = pool.alloc(need_rows) if need_rows else []
        if rows is None:
            raise RuntimeError("req_to_token_pool exhausted; lower max_running_requests")
        rows = list(rows)

        input_ids: list[int] = []
        prefix_lens, seq_lens, last_locs = [], [], []
        for r in reqs:
            fresh_row = r.req_pool_idx is None
            if fresh_row:
                r.req_pool_idx = rows.pop(0)
            pre = len(r.prefix_indices)
            if fresh_row or r.kv_allocated_len < pre:
                # matched (or re-matched) prefix: publish the shared slots in the request's row
                pool.write(r.req_pool_idx, 0, r.prefix_indices)
            if fresh_row and hasattr(self.tree_cache, "on_request_scheduled"):
                self.tree_cache.on_request_scheduled(r)        # clone the prefix's recurrent state
            seq = len(r.fill_ids)
            if hasattr(self.tree_cache, "on_extend_scheduled"):
                self.tree_cache.on_extend_scheduled(r, pre, seq)   # may ask for a state checkpoint inside this extend
            input_ids.extend(r.fill_ids[pre:])
            prefix_lens.append(pre)
            seq_lens.append(seq)
            last_locs.append(int(r.prefix_indices[-1]) if pre > 0 else -1)
            r.cached_tokens += pre - r.already_computed
            r.already_computed = seq
            r.is_retracted = False
            # logprob start inside this extend
            if r.return_logprob and not r.return_output_logprob_only:
                start = r.logprob_start_len if r.logprob_start_len >= 0 else len(r.origin_input_ids) - 1
                r.extend_logprob_start_len = min(max(start - pre, 0), seq - pre - 1) if seq - pre > 0 else 0
            else:
                r.extend_logprob_start_len = max(seq - pre - 1, 0)

        ext = [s - p for s, p in zip(seq_lens, prefix_lens)]
        n_tok = sum(ext)
        alloc = self.token_to_kv_pool_allocator
        out = self._evict_then(
            n_tok + len(reqs) * self.page_size,
            lambda: alloc.alloc_extend(prefix_lens, seq_lens, last_locs, n_tok, dp_rank=self.dp_rank))
        if out is None:
            raise RuntimeError(
                f"Prefill out of memory: need {n_tok} tokens, "
                f"available {alloc.available_size(dp_rank=self.dp_rank)}")
        o = 0
        for r, p, s, e in zip(reqs, prefix_lens, seq_lens, ext):
            pool.write(r.req_pool_idx, p, out[o:o + e])
            r.kv_allocated_len = s
            r.kv_committed_len = s
            o += e

        self.input_ids = np.asarray(input_ids, dtype=np.int32)
        self.req_pool_indices = np.asarray([r.req_pool_idx for r in reqs], dtype=np.int32)
        self.seq_lens = np.asarray(seq_lens, dtype=np.int32)
        self.out_cache_loc = out.astype(np.int32)
        self.prefix_lens = prefix_lens
        self.extend_lens = ext
        self.extend_num_tokens = n_tok
        self.extend_logprob_start_lens = [r.extend_logprob_start_len for r in reqs]

    def mix_with_running(self, running_batch: "ScheduleBatch"):
        """Append the running decode requests to this prefill step (`--enable-mixed-chunk`,
        reference :1085-1175).  Decode rows become 1-token extends at the tail."""
        running_batch.prepare_for_decode()
        self.forward_mode = ForwardMode.MIXED
        n_dec = len(running_batch.reqs)
        self.input_ids = np.concatenate([self.input_ids, running_batch.input_ids])
        self.out_cache_loc = np.concatenate([self.out_cache_loc, running_batch.out_cache_loc])
        self.req_pool_indices = np.concatenate([self.req_pool_indices, running_batch.req_pool_indices])
        self.seq_lens = np.concatenate([self.seq_lens, running_batch.seq_lens])
        self.prefix_lens = self.prefix_lens + [int(s) - 1 for s in running_batch.seq_lens]
        self.extend_lens = self.extend_lens + [1] * n_dec
        self.extend_num_tokens += n_dec
        self.extend_logprob_start_lens = self.extend_logprob_start_lens + [0] * n_dec
        self.decoding_reqs = list(running_batch.reqs)
        self.num_decode_in_mixed = n_dec
        self.reqs = self.reqs + running_batch.reqs
        self.return_logprob = self.return_logprob or running_batch.return_logprob
        self.has_stream = self.has_stream or running_batch.has_stream
        self.has_grammar = self.has_grammar or running_batch.has_grammar

    # ------------------------------------------------------------------ decode
    # KV slots a speculative step reserves per request (set by the scheduler)
    spec_alloc_len: int = 0

    def new_page_count_next_decode(self) -> int:
        ps = self.page_size
        if self.spec_algorithm is not None and self.spec_alloc_len:
            n = self.spec_alloc_len
            return sum((r.kv_committed_len % ps + n + ps - 1) // ps for r in self.reqs)
        if ps == 1:
            return len(self.reqs)
        return sum(1 for r in self.reqs if r.kv_committed_len % ps == 0)

    def check_decode_mem(self, buf_multiplier: int = 1) -> bool:
        need = self.new_page_count_next_decode() * buf_multiplier * self.page_size
        alloc = self.token_to_kv_pool_allocator
        if alloc.available_size(dp_rank=self.dp_rank) >= need:
            return True
        if self.tree_cache is not None:
            self._cache_evict(need)
        return alloc.available_size(dp_rank=self.dp_rank) >= need

    def retract_decode(self, server_args=None):
        """Free memory by sending requests back to the waiting queue: fewest generated
        tokens first, longest prompt breaking ties (reference :1437-1545).
        Returns (retracted, new_token_ratio, aborted)."""
        order = sorted(range(len(self.reqs)),
                       key=lambda i: (len(self.reqs[i].output_ids), -len(self.reqs[i].origin_input_ids)),
                       reverse=True)
        retracted: list[Req] = []
        aborted: list[Req] = []
        alloc = self.token_to_kv_pool_allocator
        steps = global_config.retract_decode_steps

        def enough(n_left: int) -> bool:
            need = n_left * steps if self.page_size == 1 else \
                n_left * ((steps + self.page_size - 1) // self.page_size) * self.page_size
            avail = alloc.available_size(dp_rank=self.dp_rank)
            if avail >= need:
                return True
            if self.tree_cache is not None:
                self._cache_evict(need - avail)
            return alloc.available_size(dp_rank=self.dp_rank) >= need

        first = True
        while first or not enough(len(order)):
            first = False
            if len(order) == 1:
                # not even one request fits
                if not self.check_decode_mem():
                    i = order.pop()
                    r = self.reqs[i]
                    r.to_abort = True
                    r.finished_reason = FINISH_ABORT(
                        "Out of memory: the request cannot continue even alone.", 500, "InternalServerError")
                    self._release_req(r)
                    aborted.append(r)
                break
            i = order.pop()
            r = self.reqs[i]
            retracted.append(r)
            self._release_req(r)
            r.reset_for_retract()
        keep = sorted(order)
        self.filter_batch(keep_indices=keep)
        total_decoded = sum(len(r.output_ids) for r in self.reqs)
        total_max_new = sum(r.sampling_params.max_new_tokens for r in self.reqs)
        new_ratio = (total_decoded + steps * len(self.reqs)) / (total_max_new + 1)
        return retracted, min(1.0, new_ratio), aborted

    def _release_req(self, r: Req):
        """Give back a running request's KV and row (retract / abort path)."""
        pool = self.req_to_token_pool
        alloc = self.token_to_kv_pool_allocator
        if r.req_pool_idx is None:
            return
        kv = pool.read(r.req_pool_idx, r.kv_allocated_len).copy()
        shared = r.last_matched_prefix_len
        alloc.free(kv[shared:], dp_rank=self.dp_rank)
        if self.tree_cache is not None and r.last_node is not None:
            self.tree_cache.dec_lock_ref(r.last_node)
        pool.free(r.req_pool_idx)

    def prepare_for_transferred_decode(self):
        """Requests whose prompt KV arrived from a prefill engine: they join the decode batch
        as if their prefill had just run here."""
        self.forward_mode = ForwardMode.DECODE
        for r in self.reqs:
            # the first token was sampled by the prefill engine: this engine's device-side map of latest tokens has
            # nothing for the request's row yet, so its first decode step is fed the id itself, not a placeholder
            r.host_token_pending = True
        self.req_pool_indices = np.asarray([r.req_pool_idx for r in self.reqs], dtype=np.int32)
        self.seq_lens = np.asarray([r.kv_committed_len for r in self.reqs], dtype=np.int32)
        self.output_ids = None
        self.input_ids = None
        self.out_cache_loc = None
        self.prefix_lens, self.extend_lens, self.extend_num_tokens = [], [], 0
        self.num_decode_in_mixed = 0
        self.decoding_reqs = None

    def sampling_info_for_spec(self) -> ModelWorkerSamplingInfo:
        return ModelWorkerSamplingInfo.from_reqs(self.reqs, self.vocab_size)

    def prepare_for_decode(self):
        """One new token per request (reference :1680-1811)."""
        self.forward_mode = ForwardMode.DECODE
        reqs = self.reqs
        if self.spec_algorithm is not None:
            # the speculative worker reserves its own slots (several tokens per request)
            self.input_ids = np.empty(0, np.int32)
            self.output_ids = None
            self.req_pool_indices = np.asarray([r.req_pool_idx for r in reqs], dtype=np.int32)
            self.seq_lens = np.asarray([r.kv_committed_len for r in reqs], dtype=np.int32)
            self.out_cache_loc = np.empty(0, np.int32)
            self.prefix_lens, self.extend_lens, self.extend_num_tokens = [], [], 0
            self.num_decode_in_mixed = 0
            self.decoding_reqs = None
            return
        pool = self.req_to_token_pool
        alloc = self.token_to_kv_pool_allocator
        if self.enable_overlap and hasattr(alloc, "build_decode_step") and not hasattr(self.tree_cache, "evict_req_swa") \
                and pool.req_to_token.flags["C_CONTIGUOUS"]:
            # native fast path: slot choice, request -> slot table writes, positions, future-token placeholders and
            # page-table deltas of the whole batch in one C++ call
            rows = np.fromiter((r.req_pool_idx for r in reqs), np.int32, len(reqs))
            lens = np.fromiter((r.kv_committed_len for r in reqs), np.int32, len(reqs))
            built = alloc.build_decode_step(pool.req_to_token, rows, lens)
            if built is None:
                if self.tree_cache is not None:
                    self._cache_evict(len(reqs) * self.page_size)
                built = alloc.build_decode_step(pool.req_to_token, rows, lens)
                if built is None:
                    raise RuntimeError("Decode out of memory. Try to lower your batch size.")
            out, new_lens, _positions, placeholders, d_rows, d_pos, _d_ids = built
            for r_, p_ in zip(d_rows.tolist(), d_pos.tolist()):
                pool._dirty.append((r_, p_, p_ + 1))
            for i, r in enumerate(reqs):
                r.kv_committed_len += 1
                r.kv_allocated_len = r.kv_committed_len
                if r.host_token_pending:
                    placeholders[i] = r.output_ids[-1]
                    r.host_token_pending, r.penalty_restart = False, True
                    if getattr(r, "pd_time_stats", None) is not None:
                        r.pd_time_stats.mark("first_decode_step")
            self.input_ids = placeholders
            self.output_ids = None
            self.req_pool_indices = rows
            self.seq_lens = new_lens
            self.out_cache_loc = out
            self.prefix_lens = []
            self.extend_lens = []
            self.extend_num_tokens = 0
            self.num_decode_in_mixed = 0
            self.decoding_reqs = None
            return
        if self.enable_overlap:
            # The previous step may still be in flight: feed placeholders `-(row + 1)`.  The
            # future-token map slot of a row always holds the latest token sampled for the
            # request that occupies the row, whether or not the host has seen it yet.
            self.input_ids = -(np.asarray([r.req_pool_idx for r in reqs], dtype=np.int32) + 1)
            for i, r in enumerate(reqs):
                if r.host_token_pending:
                    self.input_ids[i] = r.output_ids[-1]
                    r.host_token_pending, r.penalty_restart = False, True
                    if getattr(r, "pd_time_stats", None) is not None:
                        r.pd_time_stats.mark("first_decode_step")
        else:
            for r in reqs:
                if r.host_token_pending:
                    r.host_token_pending, r.penalty_restart = False, True
                    if getattr(r, "pd_time_stats", None) is not None:
                        r.pd_time_stats.mark("first_decode_step")
            self.input_ids = np.asarray([r.output_ids[-1] if r.output_ids else r.origin_input_ids[-1]
                                         for r in reqs], dtype=np.int32)
        self.output_ids = None
        if hasattr(self.tree_cache, "evict_req_swa"):
            for r in reqs:
                if r.kv_committed_len % max(self.tree_cache.sliding_window_size // 2, 1) == 0:
                    self.tree_cache.evict_req_swa(r, r.kv_committed_len)
        old_lens = np.asarray([r.kv_committed_len for r in reqs], dtype=np.int32)
        new_lens = old_lens + 1
        last_loc = np.asarray([pool.req_to_token[r.req_pool_idx, r.kv_committed_len - 1] for r in reqs],
                              dtype=np.int32)
        out = self._evict_then(len(reqs) * self.page_size,
                               lambda: alloc.alloc_decode(new_lens, last_loc, dp_rank=self.dp_rank))
        if out is None:
            raise RuntimeError("Decode out of memory. Try to lower your batch size.")
        for r, loc in zip(reqs, out):
            pool.set_one(r.req_pool_idx, r.kv_committed_len, int(loc))
            r.kv_committed_len += 1
            r.kv_allocated_len = r.kv_committed_len
        self.req_pool_indices = np.asarray([r.req_pool_idx for r in reqs], dtype=np.int32)
        self.seq_lens = new_lens
        self.out_cache_loc = out.astype(np.int32)
        self.prefix_lens = []
        self.extend_lens = []
        self.extend_num_tokens = 0
        self.num_decode_in_mixed = 0
        self.decoding_reqs = None

    # ------------------------------------------------------------------ filter / merge
    def filter_batch(self, chunked_req_to_exclude: Req | list[Req] | None = None,
                     keep_indices: list[int] | None = None):
        if keep_indices is None:
            excl = chunked_req_to_exclude
            if excl is None:
                excl = []
            elif isinstance(excl, Req):
                excl = [excl]
            keep_indices = [i for i, r in enumerate(self.reqs) if not r.finished() and r not in excl]
        if len(keep_indices) == len(self.reqs):
            return
        idx = np.asarray(keep_indices, dtype=np.int64)
        self.reqs = [self.reqs[i] for i in keep_indices]
        for name in ("req_pool_indices", "seq_lens", "output_ids"):
            v = getattr(self, name)
            if v is not None and len(v) >= (idx.max() + 1 if len(idx) else 0):
                setattr(self, name, np.asarray(v)[idx])
        self.input_ids = None
        self.out_cache_loc = None
        self.return_logprob = any(r.return_logprob for r in self.reqs)
        self.has_stream = any(r.stream for r in self.reqs)
        self.has_grammar = any(r.grammar is not None for r in self.reqs)
        if self.batch_is_full and len(keep_indices) < len(idx) + 1:
            self.batch_is_full = False

    def merge_batch(self, other: "ScheduleBatch"):
        def cat(a, b):
            if a is None or b is None:
                return None
            return np.concatenate([np.asarray(a), np.asarray(b)])

        self.req_pool_indices = cat(self.req_pool_indices, other.req_pool_indices)
        self.seq_lens = cat(self.seq_lens, other.seq_lens)
        self.output_ids = cat(self.output_ids, other.output_ids)
        self.input_ids = None
        self.out_cache_loc = None
        self.reqs.extend(other.reqs)
        self.return_logprob |= other.return_logprob
        self.has_stream |= other.has_stream
        self.has_grammar |= other.has_grammar

    # ------------------------------------------------------------------ snapshot
    def get_model_worker_batch(self) -> ModelWorkerBatch:
        mode = self.forward_mode
        if mode.is_extend():
            pre = np.asarray(self.prefix_lens, np.int32)
            ext = np.asarray(self.extend_lens, np.int32)
            positions = np.concatenate([np.arange(p, p + e, dtype=np.int32) for p, e in zip(pre, ext)]) \
                if len(pre) else np.empty(0, np.int32)
        else:
            pre = ext = None
            positions = (self.seq_lens - 1).astype(np.int32)
        rows, pos, ids = self.req_to_token_pool.take_page_deltas()
        mm_embeds, mm_rows, mrope, deepstack = self._multimodal_inputs(positions)
        sinfo = ModelWorkerSamplingInfo.from_reqs(self.reqs, self.vocab_size)
        if mode != ForwardMode.MIXED:
            from ..sampling.penaltylib import PenaltyInfo
            sinfo.penalties = PenaltyInfo.from_reqs(self.reqs, self.seq_lens, mode.is_extend())
        return ModelWorkerBatch(
            bid=_next_bid(), forward_mode=mode, input_ids=self.input_ids,
            req_pool_indices=self.req_pool_indices, seq_lens=self.seq_lens.astype(np.int32),
            out_cache_loc=self.out_cache_loc, positions=positions,
            extend_prefix_lens=pre, extend_seq_lens=ext,
            extend_logprob_start_lens=np.asarray(self.extend_logprob_start_lens, np.int32) if mode.is_extend() else None,
            page_delta_rows=rows, page_delta_pos=pos, page_delta_ids=ids,
            sampling_info=sinfo, return_logprob=self.return_logprob,
            top_logprobs_nums=[r.top_logprobs_num for r in self.reqs] if self.return_logprob else None,
            token_ids_logprobs=[r.token_ids_logprob for r in self.reqs] if self.return_logprob else None,
            return_output_logprob_only=all(r.return_output_logprob_only or not r.return_logprob for r in self.reqs),
            capture_hidden_mode=1 if self.return_hidden_states else 0,
            return_routed_experts=any(r.return_routed_experts for r in self.reqs),
            lora_ids=[r.lora_id for r in self.reqs],
            num_decode_in_mixed=self.num_decode_in_mixed,
            spec_info=self.spec_info, spec_algorithm=self.spec_algorithm,
            dp_rank=self.dp_rank, real_bs=len(self.reqs),
            input_embeds=mm_embeds, input_embeds_rows=mm_rows, mrope_positions=mrope, deepstack_embeds=deepstack,
            recurrent_copies=(self.tree_cache.take_recurrent_copies()
                              if hasattr(self.tree_cache, "take_recurrent_copies") else None) or None,
            recurrent_tracks=(self.tree_cache.take_recurrent_tracks(self.reqs)
                              if self.forward_mode.is_extend() and hasattr(self.tree_cache, "take_recurrent_tracks")
                              else None) or None,
        )

    def _multimodal_inputs(self, positions: np.ndarray):
        """Per-token encoder embeddings and 3-D rotary positions of the requests that carry
        `mm_inputs` (reference `schedule_batch.py:2139-2230`).  Prompt tokens take their slice of
        the request's arrays; generated tokens advance all three position streams together from
        `token index + mrope_position_delta`."""
        if not any(getattr(r, "mm_inputs", None) for r in self.reqs):
            return None, None, None, None
        import torch
        T = len(positions)
        deep = None
        mrope = np.repeat(positions[None, :].astype(np.int32), 3, axis=0)
        embeds, rows = None, np.zeros(T, bool)
        if self.forward_mode.is_extend():
            offs = np.concatenate([[0], np.cumsum(self.extend_lens)]).astype(int)
            spans = [(int(offs[i]), int(self.prefix_lens[i]), int(self.extend_lens[i])) for i in range(len(self.reqs))]
        else:
            spans = [(i, int(self.seq_lens[i]) - 1, 1) for i in range(len(self.reqs))]
        for r, (off, start, n) in zip(self.reqs, spans):
            mm = getattr(r, "mm_inputs", None)
            if not mm:
                continue
            plen = len(r.origin_input_ids)
            mp = mm.get("mrope_positions")
            delta = int(mm.get("mrope_position_delta", 0) or 0)
            for j in range(n):
                p = start + j
                if mp is not None and p < plen:
                    mrope[:, off + j] = np.asarray(mp)[:, p]
                else:
                    mrope[:, off + j] = p + delta
            emb = mm.get("input_embedding")
            if emb is not None and start < plen and self.forward_mode.is_extend():
                emb = torch.as_tensor(emb)
                m = min(n, plen - start)
                if embeds is None:
                    embeds = torch.zeros(T, emb.shape[-1], dtype=emb.dtype)
                embeds[off:off + m] = emb[start:start + m]
                rows[off:off + m] = True
                ds = mm.get("deepstack")                  # [L, prompt_len, hidden], zero off the vision tokens
                if ds is not None:
                    ds = torch.as_tensor(ds)
                    if deep is None:
                        deep = torch.zeros(ds.shape[0], T, ds.shape[-1], dtype=ds.dtype)
                    deep[:, off:off + m] = ds[:, start:start + m]
        return embeds, (rows if embeds is not None else None), mrope, deep

    def copy(self) -> "ScheduleBatch":
        """Shallow snapshot used by the overlap loop to process results one step late."""
        b = ScheduleBatch(list(self.reqs), self.req_to_token_pool, self.token_to_kv_pool_allocator,
                          self.tree_cache, self.vocab_size, self.enable_overlap, self.page_size,
                          self.spec_algorithm, self.dp_rank)
        b.forward_mode = self.forward_mode
        b.prefix_lens = list(self.prefix_lens)
        b.extend_lens = list(self.extend_lens)
        b.extend_logprob_start_lens = list(self.extend_logprob_start_lens)
        b.decoding_reqs = self.decoding_reqs
        b.num_decode_in_mixed = self.num_decode_in_mixed
        b.chunked_req = self.chunked_req
        b.return_logprob = self.return_logprob
        b.seq_lens = self.seq_lens
        return b

    def __repr__(self):
        return f"ScheduleBatch(mode={self.forward_mode}, #req={len(self.reqs)})"
