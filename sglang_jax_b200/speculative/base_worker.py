"""Common plumbing of the speculative workers.

The draft model runs in its own `ModelRunner` that shares the target's request-row table
and KV slot allocator (a draft KV entry lives at the same slot index as the target entry
of the same position) and owns its own KV tensors.  Per-request draft state — the last
verified token, the hidden state that conditions the next proposal and the cached first
level of candidates — lives in device tensors indexed by the request's row, so batches
can be filtered and merged by the scheduler without touching it.

Reference: `python/sgl_jax/srt/speculative/base_worker.py`.
"""

from __future__ import annotations

from types import SimpleNamespace

import numpy as np
import torch

from ..configs.model_config import ModelConfig
from ..managers.schedule_batch import ForwardMode, ModelWorkerBatch
from ..model_executor.model_runner import ModelRunner
from ..parallel import state as ps
from .spec_info import SpeculativeAlgorithm

_bid = 1 << 40


def _next_bid() -> int:
    global _bid
    _bid += 1
    return _bid


class SpecInput(SimpleNamespace):
    """What a draft / verify forward needs beyond the plain batch arrays.

    `input_ids` / `positions` (device tensors) replace the host arrays of the worker batch,
    `hidden_states` conditions an EAGLE head, `custom_mask [B, q, tail]` restricts attention
    inside the speculative tail, `all_logits` asks for logits of every row."""

    def __init__(self, **kw):
        kw.setdefault("input_ids", None)
        kw.setdefault("positions", None)
        kw.setdefault("hidden_states", None)
        kw.setdefault("custom_mask", None)
        kw.setdefault("all_logits", False)
        super().__init__(**kw)


class BaseSpecWorker:
    def __init__(self, server_args, target_worker, algo: SpeculativeAlgorithm):
        self.server_args = server_args
        self.target_worker = target_worker
        self.algo = algo
        self.device = target_worker.device
        self.page_size = server_args.page_size
        self.topk = int(server_args.speculative_eagle_topk)
        self.num_steps = int(server_args.speculative_num_steps)
        self.num_draft_tokens = int(server_args.speculative_num_draft_tokens)
        if self.topk == 1:
            # a chain: exactly one candidate per step
            self.num_draft_tokens = min(self.num_draft_tokens, self.num_steps + 1)
        n_cand = self.topk + (self.num_steps - 1) * self.topk * self.topk
        self.num_draft_tokens = min(self.num_draft_tokens, n_cand + 1)
        # KV slots reserved per request and step (reference ALLOC_LEN_PER_DECODE)
        self.alloc_len = max((self.num_steps - 1) * self.topk, self.num_draft_tokens)
        tr = target_worker.model_runner
        self.target_runner: ModelRunner = tr
        self.req_to_token_pool = tr.req_to_token_pool
        self.greedy_only = False
        self.accept_threshold_single = float(server_args.speculative_accept_threshold_single)
        self.accept_threshold_acc = float(server_args.speculative_accept_threshold_acc)
        self.pending_deltas = None
        self.gen = torch.Generator(device="cpu")
        self.gen.manual_seed(int(server_args.random_seed or 0) + 7919)

    # ------------------------------------------------------------------ helpers
    def make_batch(self, mode: ForwardMode, rows: np.ndarray, seq_lens: np.ndarray, out_cache_loc: np.ndarray,
                   extend_prefix_lens: np.ndarray | None, extend_seq_lens: np.ndarray | None,
                   spec: SpecInput, capture_hidden_mode: int, n_tokens: int,
                   input_ids: np.ndarray | None = None, positions: np.ndarray | None = None) -> ModelWorkerBatch:
        if self.pending_deltas is not None:
            d_rows, d_pos, d_ids = self.pending_deltas       # shipped by tensor rank 0 with the step
            self.pending_deltas = None
        else:
            d_rows, d_pos, d_ids = self.req_to_token_pool.take_page_deltas()
        return ModelWorkerBatch(
            bid=_next_bid(), forward_mode=mode,
            input_ids=input_ids if input_ids is not None else np.zeros(n_tokens, np.int32),
            req_pool_indices=rows.astype(np.int32), seq_lens=seq_lens.astype(np.int32),
            out_cache_loc=out_cache_loc.astype(np.int32),
            positions=positions if positions is not None else np.zeros(n_tokens, np.int32),
            extend_prefix_lens=None if extend_prefix_lens is None else extend_prefix_lens.astype(np.int32),
            extend_seq_lens=None if extend_seq_lens is None else extend_seq_lens.astype(np.int32),
            page_delta_rows=d_rows, page_delta_pos=d_pos, page_delta_ids=d_ids,
            sampling_info=None, capture_hidden_mode=capture_hidden_mode, spec_info=spec,
            spec_algorithm=self.algo, real_bs=len(rows))


class BaseDraftWorker:
    """Owns the draft `ModelRunner` and the per-row draft state."""

    def __init__(self, server_args, target_worker, algo: SpeculativeAlgorithm, topk: int):
        self.server_args = server_args
        self.algo = algo
        self.topk = topk
        tr: ModelRunner = target_worker.model_runner
        self.target_runner = tr
        draft_path = server_args.speculative_draft_model_path or server_args.model_path
        self.model_config = ModelConfig.from_server_args(server_args, model_path=draft_path, is_draft_model=True)
        self.runner = ModelRunner(self.model_config, server_args, tr.device,
                                  req_to_token_pool=tr.req_to_token_pool, is_draft_worker=True,
                                  token_to_kv_pool=tr.token_to_kv_pool,
                                  max_total_num_tokens=tr.max_total_num_tokens)
        self.model = self.runner.model
        self.device = tr.device
        if algo.is_eagle() and hasattr(self.model, "set_embed_and_head"):
            embed, head = tr.model.get_embed_and_head()
            self.model.set_embed_and_head(embed, head)
        if algo.is_eagle3() and hasattr(tr.model, "set_eagle3_layers_to_capture"):
            tr.model.set_eagle3_layers_to_capture(getattr(self.model_config.hf_config, "eagle_aux_layers", None))
        R = tr.req_to_token_pool.size
        hd = self.model_config.hidden_size
        self.state_verified = torch.zeros(R, dtype=torch.int64, device=self.device)
        self.state_hidden = torch.zeros(R, hd, dtype=tr.dtype, device=self.device)
        self.state_topk_p = torch.zeros(R, topk, dtype=torch.float32, device=self.device)
        self.state_topk_index = torch.zeros(R, topk, dtype=torch.int64, device=self.device)

    def map_ids(self, ids: torch.Tensor) -> torch.Tensor:
        f = getattr(self.model, "map_draft_ids", None)
        return f(ids) if f is not None else ids

    def store_first_level(self, rows: torch.Tensor, logits: torch.Tensor, hidden: torch.Tensor | None,
                          verified: torch.Tensor):
        probs = torch.softmax(logits.float(), dim=-1)
        p, idx = torch.topk(probs, self.topk, dim=-1)
        self.state_topk_p[rows] = p
        self.state_topk_index[rows] = self.map_ids(idx)
        if hidden is not None:
            self.state_hidden[rows] = hidden.to(self.state_hidden.dtype)
        self.state_verified[rows] = verified.long()


def tp_size() -> int:
    return ps.get_state().tp.size
