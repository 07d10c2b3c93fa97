"""Frequency / presence penalties and `min_new_tokens` with device-resident state.

Reference: `python/sgl_jax/srt/sampling/penaltylib/` (`orchestrator.py` `BatchedPenalizerOrchestrator`,
`frequency_penalty.py`, `presence_penalty.py`, `min_new_tokens.py`): the host keeps a cumulated dense penalty per
request, adds every new token to it after each step and ships a dense `[bs, vocab]` array with every batch.

Here the state is sparse in time and lives where it is used: the model runner keeps one row of token counts per
request slot on the device (`PenaltyState`).  A decode step's input ids ARE the tokens sampled by the previous step
(already on the device, also under overlap scheduling, where the host does not know them yet), so the update is one
scatter-add of `bs` ones; the penalty is computed from the rows of the batch when the logits exist.  A batch only
carries a few numbers per row (`PenaltyInfo`), plus, for a request that (re)starts, the tokens it has generated so
far (empty for a fresh request; the whole output after a retraction).
"""

from __future__ import annotations

import dataclasses

import numpy as np
import torch


@dataclasses.dataclass
class PenaltyInfo:
    """Per-row penalty controls of one batch (host side, travels with the batch)."""
    frequency: np.ndarray            # f32 [bs]
    presence: np.ndarray             # f32 [bs]
    min_new_tokens: np.ndarray       # i32 [bs]
    generated: np.ndarray            # i32 [bs]: tokens generated before the one this step samples
    stop_ids: np.ndarray             # i32 [bs, S]: ids suppressed while generated < min_new_tokens (-1 = padding)
    restart_rows: np.ndarray         # i32 [n]: batch rows whose request (re)starts in this step (prefill)
    restart_tokens: list             # per restart row: the tokens generated so far (list of int)

    @staticmethod
    def from_reqs(reqs, seq_lens: np.ndarray, is_extend: bool, extra_stop_ids=()) -> "PenaltyInfo | None":
        """`None` when no request of the batch uses a penalty."""
        if not any(r.sampling_params.frequency_penalty or r.sampling_params.presence_penalty
                   or r.sampling_params.min_new_tokens for r in reqs):
            return None
        n = len(reqs)
        freq, pres = np.zeros(n, np.float32), np.zeros(n, np.float32)
        mnt, gen = np.zeros(n, np.int32), np.zeros(n, np.int32)
        stops = []
        for i, r in enumerate(reqs):
            sp = r.sampling_params
            freq[i], pres[i], mnt[i] = sp.frequency_penalty, sp.presence_penalty, sp.min_new_tokens
            # exact also when the host runs one step ahead of the sampled tokens: lengths are known, ids are not
            gen[i] = 0 if is_extend and not r.output_ids else max(int(seq_lens[i]) - len(r.origin_input_ids), 0)
            ids = set(sp.stop_token_ids or ()) | set(r.eos_token_ids or ()) | set(extra_stop_ids)
            tok = getattr(r, "tokenizer", None)
            if tok is not None and getattr(tok, "eos_token_id", None) is not None:
                ids.add(int(tok.eos_token_id))
            stops.append(sorted(int(x) for x in ids) if mnt[i] > 0 else [])
        width = max((len(s) for s in stops), default=0)
        stop_ids = np.full((n, max(width, 1)), -1, np.int32)
        for i, s in enumerate(stops):
            stop_ids[i, :len(s)] = s
        if is_extend:
            rows = np.arange(n, dtype=np.int32)
            toks = [list(r.output_ids) for r in reqs]
        else:
            # a request that enters decoding without a prefill here (its KV was transferred): its slot still holds the
            # previous occupant's counts.  The token fed to this step is counted by the decode update itself.
            rows = np.asarray([i for i, r in enumerate(reqs) if getattr(r, "penalty_restart", False)], np.int32)
            toks = [list(reqs[i].output_ids[:-1]) for i in rows.tolist()]
        for r in reqs:
            if getattr(r, "penalty_restart", False):
                r.penalty_restart = False
        return PenaltyInfo(freq, pres, mnt, gen, stop_ids, rows, toks)


class PenaltyState:
    """Token counts per request slot on the device (`int32 [slots, vocab]`, allocated on first use)."""

    def __init__(self, num_slots: int, vocab_size: int, device):
        self.num_slots, self.vocab_size, self.device = num_slots, vocab_size, device
        self.counts: torch.Tensor | None = None

    def _ensure(self):
        if self.counts is None:
            self.counts = torch.zeros((self.num_slots, self.vocab_size), dtype=torch.int32, device=self.device)

    @torch.no_grad()
    def apply(self, logits: torch.Tensor, info: PenaltyInfo, slots, input_ids: torch.Tensor | None,
              is_decode: bool) -> torch.Tensor:
        """Bring the counts of the batch's slots up to date and return the penalised fp32 logits `[bs, vocab]`.

        `slots`: request slot of every batch row; `input_ids` (decode): the tokens fed to this step, i.e. the ones
        the previous step sampled."""
        self._ensure()
        dev = self.device
        slots_t = torch.as_tensor(np.asarray(slots, np.int64)).to(dev)
        V = self.vocab_size
        for r, toks in zip(info.restart_rows.tolist(), info.restart_tokens):
            row = self.counts[int(slots[r])]
            row.zero_()
            if toks:
                t = torch.as_tensor(np.asarray(toks, np.int64)).to(dev).clamp_(0, V - 1)
                row.index_add_(0, t, torch.ones_like(t, dtype=torch.int32))
        if is_decode and input_ids is not None:
            ids = input_ids.reshape(-1).long().clamp(0, V - 1)
            self.counts.index_put_((slots_t, ids), torch.ones_like(ids, dtype=torch.int32), accumulate=True)
        out = logits.float()
        Vl = out.shape[-1]
        c = self.counts[slots_t][:, :Vl].float()
        freq = torch.as_tensor(info.frequency).to(dev).view(-1, 1)
        pres = torch.as_tensor(info.presence).to(dev).view(-1, 1)
        out = out - freq * c - pres * (c > 0).float()
        early = info.generated < info.min_new_tokens
        if early.any():
            ids = torch.as_tensor(info.stop_ids.astype(np.int64)).to(dev)
            rows = torch.arange(len(early), device=dev).view(-1, 1).expand_as(ids)
            keep = torch.as_tensor(early).to(dev).view(-1, 1) & (ids >= 0) & (ids < Vl)
            out[rows[keep], ids[keep]] = float("-inf")
        return out
