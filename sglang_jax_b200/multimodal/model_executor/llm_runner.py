"""A minimal generation loop over `ModelRunner` for pipeline stages whose prefill mixes token
embeddings with encoder outputs (image / audio embeddings spliced over placeholder tokens).
One request at a time, greedy or temperature sampling, paged KV through the runner's pools."""

from __future__ import annotations

import numpy as np
import torch

from ...managers.schedule_batch import ForwardMode, ModelWorkerBatch, ModelWorkerSamplingInfo


class EmbedsGenerator:
    def __init__(self, runner):
        self.runner = runner
        self.page = runner.page_size
        self.next_page = 1

    def _alloc(self, row: int, start: int, n: int) -> np.ndarray:
        """Sequential page allocation private to this generator (the stage owns the whole pool)."""
        pool = self.runner.req_to_token_pool
        P = self.page
        slots = []
        for pos in range(start, start + n):
            if pos % P == 0:
                pool.set_one(row, pos, self.next_page * P)
                self.next_page += 1
            else:
                prev = int(pool.req_to_token[row, pos - 1])
                pool.set_one(row, pos, prev + 1)
            slots.append(int(pool.req_to_token[row, pos]))
        return np.asarray(slots, np.int32)

    def _sinfo(self, temperature: float):
        t = max(float(temperature), 0.0)
        greedy = t < 1e-6
        return ModelWorkerSamplingInfo(np.full(1, 1.0 if greedy else t, np.float32), np.ones(1, np.float32),
                                       np.full(1, 1 if greedy else 1 << 30, np.int32), np.zeros(1, np.float32), None,
                                       greedy, False, False, False)

    # ------------------------------------------------------------------ stepwise API
    def begin(self, total_len: int):
        """Start a new sequence (the generator serves one at a time) that will grow to `total_len`."""
        r = self.runner
        if total_len > r.req_to_token_pool.max_context_len or total_len > r.max_total_num_tokens:
            raise ValueError("request does not fit the stage's KV pool")
        self.next_page = 1
        self.length = 0
        self.temperature = 0.0

    @torch.inference_mode()
    def extend(self, input_ids: list[int], input_embeds: torch.Tensor | None = None, capture_hidden: bool = False,
               mrope_positions: np.ndarray | None = None):
        """Prefill `len(input_ids)` positions; returns (sampled token, last hidden state or None)."""
        r, row, n, start = self.runner, 0, len(input_ids), self.length
        loc = self._alloc(row, start, n)
        rows, pos, ids = r.req_to_token_pool.take_page_deltas()
        batch = ModelWorkerBatch(
            bid=1, forward_mode=ForwardMode.EXTEND, input_ids=np.asarray(input_ids, np.int32),
            req_pool_indices=np.asarray([row], np.int32), seq_lens=np.asarray([start + n], np.int32), out_cache_loc=loc,
            positions=np.arange(start, start + n, dtype=np.int32), extend_prefix_lens=np.asarray([start], np.int32),
            extend_seq_lens=np.asarray([n], np.int32), extend_logprob_start_lens=np.zeros(1, np.int32),
            page_delta_rows=rows, page_delta_pos=pos, page_delta_ids=ids, sampling_info=self._sinfo(self.temperature),
            input_embeds=input_embeds, capture_hidden_mode=1 if capture_hidden else 0,
            mrope_positions=None if mrope_positions is None else np.asarray(mrope_positions, np.int32))
        out, tok, _ = r.forward(batch)
        self.length = start + n
        return int(tok[0]), (out.hidden_states if capture_hidden else None)

    @torch.inference_mode()
    def step(self, token_id: int, input_embed: torch.Tensor | None = None, capture_hidden: bool = False,
             mrope_delta: int | None = None):
        """Decode one position whose input is `token_id` (or `input_embed [1, hidden]`)."""
        r, row, cur = self.runner, 0, self.length
        loc = self._alloc(row, cur, 1)
        rows, pos, ids = r.req_to_token_pool.take_page_deltas()
        batch = ModelWorkerBatch(
            bid=2, forward_mode=ForwardMode.DECODE, input_ids=np.asarray([token_id], np.int32),
            req_pool_indices=np.asarray([row], np.int32), seq_lens=np.asarray([cur + 1], np.int32),
            out_cache_loc=loc, positions=np.asarray([cur], np.int32), page_delta_rows=rows, page_delta_pos=pos,
            page_delta_ids=ids, sampling_info=self._sinfo(self.temperature), input_embeds=input_embed,
            capture_hidden_mode=1 if capture_hidden else 0,
            mrope_positions=None if mrope_delta is None else np.full((3, 1), cur + mrope_delta, np.int32))
        out, tok, _ = r.forward(batch)
        self.length = cur + 1
        return int(tok[0]), (out.hidden_states if capture_hidden else None)

    def generate(self, input_ids: list[int], input_embeds: torch.Tensor | None, max_new_tokens: int = 16,
                 temperature: float = 0.0, eos_ids: set[int] | None = None,
                 mrope_positions: np.ndarray | None = None, mrope_delta: int = 0) -> list[int]:
        self.begin(len(input_ids) + max_new_tokens)
        self.temperature = temperature
        tok, _ = self.extend(input_ids, input_embeds, mrope_positions=mrope_positions)
        out = [tok]
        eos_ids = eos_ids or set()
        while len(out) < max_new_tokens and out[-1] not in eos_ids:
            tok, _ = self.step(out[-1], mrope_delta=mrope_delta if mrope_positions is not None else None)
            out.append(tok)
        return out
