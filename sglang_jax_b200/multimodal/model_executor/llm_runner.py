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

    @torch.inference_mode()
    def generate(self, input_ids: list[int], input_embeds: torch.Tensor | None, max_new_tokens: int = 16,
                 temperature: float = 0.0, eos_ids: set[int] | None = None,
                 mrope_positions: np.ndarray | None = None, mrope_delta: int = 0) -> list[int]:
        r = self.runner
        row = 0
        self.next_page = 1
        n = len(input_ids)
        total = n + max_new_tokens
        if total > r.req_to_token_pool.max_context_len or total > r.max_total_num_tokens:
            raise ValueError("request does not fit the stage's KV pool")
        loc = self._alloc(row, 0, n)
        rows, pos, ids = r.req_to_token_pool.take_page_deltas()
        batch = ModelWorkerBatch(
            bid=1, forward_mode=ForwardMode.EXTEND, input_ids=np.asarray(input_ids, np.int32),
            req_pool_indices=np.asarray([row], np.int32), seq_lens=np.asarray([n], np.int32), out_cache_loc=loc,
            positions=np.arange(n, dtype=np.int32), extend_prefix_lens=np.zeros(1, np.int32),
            extend_seq_lens=np.asarray([n], np.int32), extend_logprob_start_lens=np.zeros(1, np.int32),
            page_delta_rows=rows, page_delta_pos=pos, page_delta_ids=ids, sampling_info=self._sinfo(temperature),
            input_embeds=input_embeds,
            mrope_positions=None if mrope_positions is None else np.asarray(mrope_positions, np.int32))
        _, tok, _ = r.forward(batch)
        out = [int(tok[0])]
        eos_ids = eos_ids or set()
        while len(out) < max_new_tokens and out[-1] not in eos_ids:
            cur = n + len(out) - 1
            loc = self._alloc(row, cur, 1)
            rows, pos, ids = r.req_to_token_pool.take_page_deltas()
            batch = ModelWorkerBatch(
                bid=2, forward_mode=ForwardMode.DECODE, input_ids=np.asarray([out[-1]], np.int32),
                req_pool_indices=np.asarray([row], np.int32), seq_lens=np.asarray([cur + 1], np.int32),
                out_cache_loc=loc, positions=np.asarray([cur], np.int32), page_delta_rows=rows, page_delta_pos=pos,
                page_delta_ids=ids, sampling_info=self._sinfo(temperature),
                mrope_positions=None if mrope_positions is None else np.full((3, 1), cur + mrope_delta, np.int32))
            _, tok, _ = r.forward(batch)
            out.append(int(tok[0]))
        return out
