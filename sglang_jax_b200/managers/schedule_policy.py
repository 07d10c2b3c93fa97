"""Queue ordering and token-budget admission for prefill.

Contracts follow the reference's `python/sgl_jax/srt/managers/schedule_policy.py`
(`SchedulePolicy` :74-260, `PrefillAdder` :266-759): `lpm`/`dfs-weight` need the
radix tree, `lpm` falls back to `fcfs` above 128 waiting requests, requests that
share a long *uncached* prefix with one already picked are deprioritised so the
first one can populate the cache, extend lengths are charged rounded up to whole
pages, and an input that does not fit the chunk budget is truncated to a page
multiple and continued next step ("chunked prefill").
"""

from __future__ import annotations

import numpy as np

import random
from collections import defaultdict
from enum import Enum, auto

from ..global_config import global_config
from ..mem_cache.radix_cache import RadixCache, RadixKey
from .schedule_batch import Req

# Above this queue length LPM's per-request prefix matching costs more than it saves.
LPM_FALLBACK_QUEUE_LEN = 128
IN_BATCH_PREFIX_CACHING_CHECK_THRESHOLD = 32
IN_BATCH_PREFIX_CACHING_DEPRIORITIZE_THRESHOLD = 32
IGNORE_EOS_RESERVE_TOKENS = 1


class AddReqResult(Enum):
    CONTINUE = auto()   # keep scanning the queue
    NO_TOKEN = auto()   # KV memory exhausted for this rank
    OTHER = auto()      # per-step input / chunk budget exhausted


class SchedulePolicy:
    def __init__(self, policy: str, tree_cache, enable_hierarchical_cache: bool = False):
        if tree_cache is None or getattr(tree_cache, "disable", True):
            if policy in ("lpm", "dfs-weight"):
                policy = "fcfs"
        self.policy = policy
        self.tree_cache = tree_cache
        # scratch tree used only to detect shared uncached prefixes inside one queue
        self.waiting_queue_radix_tree = RadixCache(None, None, page_size=1, disable=False)

    def calc_priority(self, waiting_queue: list[Req]) -> bool:
        """Sorts `waiting_queue` in place; returns whether prefix matches were computed."""
        policy = self.policy
        if policy == "fcfs":
            return False
        if policy == "lpm" and len(waiting_queue) > LPM_FALLBACK_QUEUE_LEN:
            return False
        computed = False
        if policy in ("lpm", "dfs-weight"):
            deprioritized = self._compute_prefix_matches(waiting_queue)
            computed = True
            if policy == "lpm":
                waiting_queue.sort(key=lambda r: (r.rid in deprioritized, -len(r.prefix_indices)))
            else:
                self._sort_dfs_weight(waiting_queue)
        elif policy == "lof":
            waiting_queue.sort(key=lambda r: -r.sampling_params.max_new_tokens)
        elif policy == "random":
            random.shuffle(waiting_queue)
        else:
            raise ValueError(f"Unknown schedule_policy: {policy}")
        return computed

    def _compute_prefix_matches(self, waiting_queue: list[Req]) -> set[str]:
        deprioritized: set[str] = set()
        scratch = self.waiting_queue_radix_tree
        scratch.reset()
        for r in waiting_queue:
            ids = r.adjust_max_prefix_ids() if r.fill_ids else (r.origin_input_ids + r.output_ids)[:-1]
            key = RadixKey(ids, r.extra_key, r.dp_rank or 0)
            res = self.tree_cache.match_prefix(key)
            r.prefix_indices, r.last_node = res.device_indices, res.last_device_node
            r.last_matched_prefix_len = len(r.prefix_indices)
            if len(r.prefix_indices) <= IN_BATCH_PREFIX_CACHING_CHECK_THRESHOLD:
                in_batch = scratch.match_prefix(key).device_indices
                if len(in_batch) >= IN_BATCH_PREFIX_CACHING_DEPRIORITIZE_THRESHOLD:
                    deprioritized.add(r.rid)
                else:
                    scratch.insert(key)
        return deprioritized

    def _sort_dfs_weight(self, waiting_queue: list[Req]):
        by_node = defaultdict(list)
        for r in waiting_queue:
            by_node[r.last_node].append(r)
        weight = defaultdict(int)
        for node, rs in by_node.items():
            weight[node] = len(rs)

        def calc(node):
            for c in node.children.values():
                calc(c)
                weight[node] += weight[c]

        root = self.tree_cache.root_node
        calc(root)
        out: list[Req] = []

        def dfs(node):
            for c in sorted(node.children.values(), key=lambda x: -weight[x]):
                dfs(c)
            out.extend(by_node.get(node, []))

        dfs(root)
        assert len(out) == len(waiting_queue)
        waiting_queue[:] = out


class PrefillAdder:
    """Admits waiting requests into one prefill step under three budgets:
    total KV tokens (`rem_total_tokens`), per-step input tokens (`rem_input_tokens`)
    and the chunk size (`rem_chunk_tokens`)."""

    def __init__(self, page_size: int, tree_cache, token_to_kv_pool_allocator, running_batch,
                 new_token_ratio: float, rem_input_tokens: int, rem_chunk_tokens: int | None,
                 mixed_with_decode_tokens: int = 0, dp_rank: int = 0):
        self.page_size = page_size
        self.tree_cache = tree_cache
        self.alloc = token_to_kv_pool_allocator
        self.running_batch = running_batch
        self.new_token_ratio = new_token_ratio
        self.dp_rank = dp_rank
        self.rem_input_tokens = rem_input_tokens - mixed_with_decode_tokens
        self.rem_chunk_tokens = rem_chunk_tokens
        if self.rem_chunk_tokens is not None:
            self.rem_chunk_tokens -= mixed_with_decode_tokens
        self.rem_total_token_offset = mixed_with_decode_tokens
        self.cur_rem_token_offset = mixed_with_decode_tokens
        self.req_states = None
        self.can_run_list: list[Req] = []
        self.new_chunked_req: Req | None = None
        self.log_hit_tokens = 0
        self.log_input_tokens = 0
        if running_batch is not None:
            clip = global_config.clip_max_new_tokens_estimation
            self.rem_total_token_offset += sum(
                min(r.sampling_params.max_new_tokens - len(r.output_ids), clip) * new_token_ratio
                for r in running_batch.reqs)

    # budgets ------------------------------------------------------------
    def _pool_tokens(self) -> int:
        ev = self.tree_cache.evictable_size(self.dp_rank) if self.tree_cache is not None else 0
        return self.alloc.available_size(dp_rank=self.dp_rank) + ev

    @property
    def rem_total_tokens(self) -> int:
        return int(self._pool_tokens() - self.rem_total_token_offset)

    @property
    def cur_rem_tokens(self) -> int:
        return int(self._pool_tokens() - self.cur_rem_token_offset)

    def ceil_paged_tokens(self, n: int) -> int:
        return -(-n // self.page_size) * self.page_size

    def budget_state(self) -> AddReqResult:
        if self.rem_total_tokens <= 0 or self.cur_rem_tokens <= 0:
            return AddReqResult.NO_TOKEN
        if self.rem_input_tokens <= 0 or (self.rem_chunk_tokens is not None and self.rem_chunk_tokens <= 0):
            return AddReqResult.OTHER
        return AddReqResult.CONTINUE

    def _update_prefill_budget(self, prefix_len: int, extend_input_len: int, max_new_tokens: int):
        extend_input_len = self.ceil_paged_tokens(extend_input_len)
        self.rem_total_token_offset += extend_input_len + max_new_tokens
        self.cur_rem_token_offset += extend_input_len
        self.rem_input_tokens -= extend_input_len
        if self.rem_chunk_tokens is not None:
            self.rem_chunk_tokens -= extend_input_len
        self.log_hit_tokens += prefix_len
        self.log_input_tokens += extend_input_len

    # chunk continuation ---------------------------------------------------
    def add_chunked_req(self, req: Req) -> Req | None:
        budget = min(self.rem_chunk_tokens, self.rem_total_tokens) if self.rem_chunk_tokens is not None \
            else self.rem_total_tokens
        if budget <= 0:
            budget = self.rem_chunk_tokens if self.rem_chunk_tokens is not None else req.extend_input_len
        truncated = req.extend_input_len > budget
        if truncated:
            budget = budget // self.page_size * self.page_size
            req.extend_input_len = budget
            req.fill_ids = req.fill_ids[: len(req.prefix_indices) + req.extend_input_len]
        self.can_run_list.append(req)
        self._update_prefill_budget(
            0, req.extend_input_len,
            0 if truncated else min(req.sampling_params.max_new_tokens,
                                    global_config.clip_max_new_tokens_estimation))
        return req if truncated else None

    # ignore-eos fast path ---------------------------------------------------
    def add_one_req_ignore_eos(self, req: Req) -> AddReqResult:
        """With `ignore_eos` every request runs to `max_new_tokens`, so future frees are
        known: simulate them to check the new request never starves the pool
        (reference :537-622)."""
        def tokens_left(r: Req) -> int:
            return r.sampling_params.max_new_tokens - len(r.output_ids)

        if self.ceil_paged_tokens(req.extend_input_len) > min(self.cur_rem_tokens, self.rem_total_tokens):
            return AddReqResult.NO_TOKEN
        if self.req_states is None:
            self.req_states = []
            if self.running_batch is not None:
                for r in self.running_batch.reqs:
                    self.req_states.append((tokens_left(r), r.seqlen))
            for r in self.can_run_list:
                self.req_states.append((tokens_left(r), r.extend_input_len))
            self.req_states.sort(key=lambda x: x[0])
        new_state = (tokens_left(req), req.extend_input_len)
        import bisect
        states = list(self.req_states)
        bisect.insort(states, new_state, key=lambda x: x[0])
        cur_rem = self.cur_rem_tokens - self.ceil_paged_tokens(req.extend_input_len)
        prev_left = 0
        for i, (left, occupied) in enumerate(states):
            # the remaining (len - i) requests each decode (left - prev_left) more tokens
            decode_steps = left - prev_left
            cur_rem -= (len(states) - i) * decode_steps
            if cur_rem < IGNORE_EOS_RESERVE_TOKENS and decode_steps > 0:
                return AddReqResult.NO_TOKEN
            cur_rem += occupied + left   # request i finishes and frees everything it held
            prev_left = left
        self.req_states = states
        if self.rem_chunk_tokens is None or req.extend_input_len <= self.rem_chunk_tokens:
            self.can_run_list.append(req)
            self._update_prefill_budget(0, req.extend_input_len,
                                        min(req.sampling_params.max_new_tokens,
                                            global_config.clip_max_new_tokens_estimation))
        else:
            if self.rem_chunk_tokens <= 0:
                return AddReqResult.OTHER
            trunc = self.rem_chunk_tokens // self.page_size * self.page_size
            if trunc <= 0:
                return AddReqResult.OTHER
            req.extend_input_len = trunc
            req.fill_ids = req.fill_ids[:trunc]
            self.can_run_list.append(req)
            self.new_chunked_req = req
            self._update_prefill_budget(0, trunc, 0)
        return self.budget_state()

    # normal path ----------------------------------------------------------------
    def add_one_req(self, req: Req) -> AddReqResult:
        cache_disabled = self.tree_cache is None or getattr(self.tree_cache, "disable", True)
        if req.sampling_params.ignore_eos and cache_disabled:
            return self.add_one_req_ignore_eos(req)
        clip = global_config.clip_max_new_tokens_estimation
        if req.host_hit_length > 0 and hasattr(self.tree_cache, "init_load_back"):
            # part of the prefix lives on the host tier: give it device slots and start the copy
            new_indices, new_last = self.tree_cache.init_load_back(req.last_host_node, req.host_hit_length)
            req.host_hit_length = 0
            if len(new_indices):
                req.prefix_indices = np.concatenate([req.prefix_indices, new_indices]).astype(np.int32)
                req.last_node = new_last
                req.last_matched_prefix_len = len(req.prefix_indices)
                req.extend_input_len = len(req.fill_ids) - len(req.prefix_indices)
        total_tokens = req.extend_input_len + min(req.sampling_params.max_new_tokens, clip)
        if total_tokens >= self.rem_total_tokens:
            return AddReqResult.NO_TOKEN
        input_tokens = self.ceil_paged_tokens(req.extend_input_len)
        if input_tokens >= self.rem_input_tokens and len(self.can_run_list) != 0:
            return AddReqResult.OTHER
        # Lock the matched branch while deciding so eviction (triggered by our own
        # budget arithmetic) cannot take it away.
        tc = self.tree_cache
        if not cache_disabled:
            tc.inc_lock_ref(req.last_node)
        try:
            if total_tokens >= self.rem_total_tokens:
                return AddReqResult.NO_TOKEN
            prefix_len = len(req.prefix_indices)
            if self.rem_chunk_tokens is None or input_tokens <= self.rem_chunk_tokens:
                # whole remaining input fits
                self.can_run_list.append(req)
                if not cache_disabled:
                    tc.inc_lock_ref(req.last_node)
                self._update_prefill_budget(prefix_len, req.extend_input_len,
                                            min(req.sampling_params.max_new_tokens, clip))
            else:
                trunc = self.rem_chunk_tokens // self.page_size * self.page_size
                if trunc <= 0:
                    return AddReqResult.OTHER
                req.extend_input_len = trunc
                req.fill_ids = req.fill_ids[: prefix_len + trunc]
                self.can_run_list.append(req)
                self.new_chunked_req = req
                if not cache_disabled:
                    tc.inc_lock_ref(req.last_node)
                self._update_prefill_budget(prefix_len, trunc, 0)
        finally:
            if not cache_disabled:
                tc.dec_lock_ref(req.last_node)
        return self.budget_state()
