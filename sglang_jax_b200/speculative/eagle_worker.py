"""Orchestration of one speculative step: draft -> verify -> draft-extend.

Reference: `python/sgl_jax/srt/speculative/eagle_worker.py` (verify + orchestration),
scheduler hook `python/sgl_jax/srt/managers/scheduler.py:2617-2722`.

Prefill: the target runs the usual EXTEND with all hidden states captured; the draft then
extends over the same tokens shifted left by one (the sampled token closes the sequence).

Decode, per request with `L` cached tokens:
  1. reserve `alloc_len` KV slots behind position `L`;
  2. `draft()` grows a candidate tree, `build_tree` keeps the best `num_draft_tokens - 1`;
  3. the target scores the whole tree in one TARGET_VERIFY forward (ancestor mask);
  4. greedy or stochastic acceptance walks the tree; accepted nodes' KV entries are moved
     to the front of the reservation so the cache stays position-contiguous;
  5. the draft re-runs the accepted tokens with the target's hidden states.
The scheduler appends the accepted tokens, then returns the unused tail of the reservation.
"""

from __future__ import annotations

import logging
import os

import numpy as np
import torch

from ..managers.schedule_batch import ForwardMode, ScheduleBatch
from ..managers.tp_worker import GenerationBatchResult
from ..ops import reference
from .base_worker import BaseSpecWorker, SpecInput
from .eagle_draft_worker import EagleDraftWorker
from .eagle_util import build_tree, tree_speculative_sampling_target_only, verify_tree_greedy
from .spec_info import SpeculativeAlgorithm
from .spec_utils import simulated_accept_len

logger = logging.getLogger(__name__)


class EAGLEWorker(BaseSpecWorker):
    def __init__(self, server_args, target_worker, algo: SpeculativeAlgorithm):
        super().__init__(server_args, target_worker, algo)
        if algo.is_nextn():
            from .multi_layer_draft_worker import MultiLayerDraftWorker
            self.draft_worker = MultiLayerDraftWorker(server_args, target_worker, algo, self)
        else:
            self.draft_worker = EagleDraftWorker(server_args, target_worker, algo, self)
        self.uses_aux = algo.is_eagle3()
        self.sim_acc = simulated_accept_len()
        logger.info("speculative decoding: %s, steps=%d topk=%d draft_tokens=%d", algo.name, self.num_steps,
                    self.topk, self.num_draft_tokens)

    # ------------------------------------------------------------------ entry
    def forward_batch_speculative_generation(self, batch: ScheduleBatch) -> GenerationBatchResult:
        if batch.forward_mode.is_extend():
            return self._prefill(batch)
        return self._decode(batch)

    # ------------------------------------------------------------------ prefill
    def _target_hidden(self, out) -> torch.Tensor:
        if self.uses_aux:
            return torch.cat(out.extras["aux_hidden_states"], dim=-1)
        return out.hidden_states

    def _prefill(self, batch: ScheduleBatch) -> GenerationBatchResult:
        mwb = batch.get_model_worker_batch()
        assert mwb.num_decode_in_mixed == 0, "mixed chunks are not combined with speculative decoding"
        # the token after a non-final chunk is the next prompt token
        chunk_next = np.full(len(batch.reqs), -1, np.int64)
        for i, r in enumerate(batch.reqs):
            full_len = len(r.origin_input_ids) + len(r.output_ids)
            end = len(r.fill_ids)
            if end < full_len:
                chunk_next[i] = (r.origin_input_ids + r.output_ids)[end]
        self.target_worker.spec_broadcast("spec_prefill", (mwb, chunk_next, batch.return_hidden_states))
        return self.prefill_core(mwb, chunk_next, batch.return_hidden_states)

    @torch.inference_mode()
    def prefill_core(self, mwb, chunk_next: np.ndarray, want_hidden: bool = False) -> GenerationBatchResult:
        """Runs on every tensor rank with the same host inputs."""
        mwb.capture_hidden_mode = 2
        res = self.target_worker.forward_batch_generation(mwb, broadcast=False)
        out = res.logits_output
        self.draft_worker.draft_extend_for_prefill(mwb, res.next_token_ids, self._target_hidden(out), chunk_next)
        if want_hidden and out.hidden_states is not None:
            last = torch.from_numpy(np.cumsum(np.asarray(mwb.extend_seq_lens)) - 1).to(self.device).long()
            out.hidden_states = out.hidden_states[last]
        else:
            out.hidden_states = None
        return res

    # ------------------------------------------------------------------ decode
    def _reserve(self, batch: ScheduleBatch):
        reqs = batch.reqs
        pool = self.req_to_token_pool
        alloc = batch.token_to_kv_pool_allocator
        L = np.asarray([r.kv_committed_len for r in reqs], dtype=np.int32)
        rows = np.asarray([r.req_pool_idx for r in reqs], dtype=np.int32)
        last_loc = np.asarray([pool.req_to_token[r.req_pool_idx, r.kv_committed_len - 1] for r in reqs], np.int32)
        n = self.alloc_len
        out = batch._evict_then(len(reqs) * (n + self.page_size),
                                lambda: alloc.alloc_extend(L, L + n, last_loc, len(reqs) * n, dp_rank=batch.dp_rank))
        if out is None:
            raise RuntimeError("speculative decode out of KV memory; lower the batch size or the draft size")
        tail = np.asarray(out, np.int32).reshape(len(reqs), n)
        for b, r in enumerate(reqs):
            pool.write(r.req_pool_idx, int(L[b]), tail[b])
            r.kv_allocated_len = int(L[b]) + n
        return rows, L, tail

    def _decode(self, batch: ScheduleBatch) -> GenerationBatchResult:
        rows_np, L, tail = self._reserve(batch)
        deltas = self.req_to_token_pool.take_page_deltas()
        sinfo = batch.sampling_info_for_spec()
        self.target_worker.spec_broadcast("spec_decode", (rows_np, L, tail, deltas, sinfo))
        return self.decode_core(rows_np, L, tail, deltas, sinfo)

    @torch.inference_mode()
    def decode_core(self, rows_np, L, tail, deltas, sinfo) -> GenerationBatchResult:
        """Runs on every tensor rank with the same host inputs (slots were reserved by rank 0)."""
        dw = self.draft_worker
        dev = self.device
        self.pending_deltas = deltas
        B = len(rows_np)
        rows = torch.from_numpy(rows_np.astype(np.int64)).to(dev)
        S = self.num_steps

        cand_tok, cand_score, cand_parent = dw.draft(rows_np, L, tail)
        verified = dw.state_verified[rows]
        tokens, parent, depth, mask, _ = build_tree(verified, cand_tok, cand_score, cand_parent,
                                                    self.num_draft_tokens, S)
        n = tokens.shape[1]

        # ---- verify
        L_t = torch.from_numpy(L.astype(np.int64)).to(dev)
        pos = (L_t.view(B, 1) + depth).reshape(-1)
        spec = SpecInput(input_ids=tokens.reshape(-1).int(), positions=pos.int(), all_logits=True,
                         custom_mask=None if self.topk == 1 else mask)
        vb = self.make_batch(ForwardMode.TARGET_VERIFY, rows_np, L + n, tail[:, :n].reshape(-1), L,
                             np.full(B, n, np.int32), spec, 2, B * n)
        out, _, _ = self.target_runner.forward(vb, skip_sample=True)
        logits = out.next_token_logits.view(B, n, -1)
        if sinfo.is_all_greedy:
            target_ids = logits.argmax(dim=-1)
            accept, path, bonus = verify_tree_greedy(tokens, parent, target_ids, S)
        else:
            accept, path, bonus = self._stochastic_verify(tokens, parent, logits, sinfo, S)
        if self.sim_acc is not None:
            accept, path = self._force_accept(accept, path, parent, n)
        accept = accept.clamp_max(n - 1)

        # ---- host view of the outcome (one sync per step, as in the plain decode loop)
        acc_np = accept.cpu().numpy().astype(np.int64)
        path_np = path.cpu().numpy()
        tok_np = tokens.cpu().numpy()
        bonus_np = bonus.cpu().numpy()
        out_tokens: list[list[int]] = []
        src_slots, dst_slots = [], []
        flat_idx = []
        for b in range(B):
            a = int(acc_np[b])
            chain = path_np[b, :a + 1]
            out_tokens.append([int(tok_np[b, j]) for j in chain[1:]] + [int(bonus_np[b])])
            for i, j in enumerate(chain):
                flat_idx.append(b * n + int(j))
                if int(j) != i:
                    src_slots.append(tail[b, int(j)])
                    dst_slots.append(tail[b, i])
        if src_slots:
            self.target_runner.token_to_kv_pool.move_kv(
                torch.tensor(src_slots, dtype=torch.long, device=dev),
                torch.tensor(dst_slots, dtype=torch.long, device=dev))

        # ---- draft extend over the accepted chain
        flat = torch.tensor(flat_idx, dtype=torch.long, device=dev)
        hidden = self._target_hidden(out)[flat] if dw.uses_hidden else None
        new_tokens = torch.tensor([t for ts in out_tokens for t in ts], dtype=torch.long, device=dev)
        dw.draft_extend_after_verify(rows_np, L, acc_np, tail, new_tokens, hidden, bonus)

        res = GenerationBatchResult(None, None, bid=vb.bid)
        res.spec_tokens = out_tokens
        res.accept_lens = acc_np
        res.alloc_ends = (L + self.alloc_len).astype(np.int64)
        return res

    # ------------------------------------------------------------------ acceptance
    def _stochastic_verify(self, tokens, parent, logits, sinfo, S):
        B, n, V = logits.shape
        dev = logits.device
        rep = lambda a, d: torch.as_tensor(np.asarray(a), dtype=d).to(dev).repeat_interleave(n)
        probs = reference.top_k_top_p_min_p_probs(
            logits.reshape(B * n, V).float(), rep(sinfo.temperatures, torch.float32),
            rep(sinfo.top_ks, torch.int64), rep(sinfo.top_ps, torch.float32), rep(sinfo.min_ps, torch.float32))
        coins = torch.rand(B, S + 1, generator=self.gen).to(dev)
        final = torch.rand(B, generator=self.gen).to(dev)
        return tree_speculative_sampling_target_only(tokens, parent, probs.view(B, n, V), coins, final, S,
                                                     self.accept_threshold_single, self.accept_threshold_acc)

    def _force_accept(self, accept, path, parent, n):
        """Benchmark aid: pretend the first chain of the tree was accepted up to a fixed
        length (the emitted tokens are then not the target's)."""
        want = min(int(self.sim_acc), path.shape[1] - 1, n - 1)
        B = accept.shape[0]
        cur = torch.zeros(B, dtype=torch.long, device=accept.device)
        new_path = torch.full_like(path, -1)
        new_path[:, 0] = 0
        got = torch.zeros_like(accept)
        for d in range(1, want + 1):
            child = (parent == cur.view(B, 1))
            child[:, 0] = False
            has = child.any(1)
            nxt = child.float().argmax(1)
            cur = torch.where(has, nxt, cur)
            new_path[:, d] = torch.where(has, nxt, torch.full_like(nxt, -1))
            got += has.long()
        return got, new_path
