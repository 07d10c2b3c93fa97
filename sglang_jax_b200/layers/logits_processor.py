"""Hidden states -> logits (+ logprobs).

Reference: `python/sgl_jax/srt/layers/logits_processor.py` (`LogitsProcessorOutput` :27,
`LogitsMetadata` :97, `LogitsProcessor` :249, `_get_logits` :523).  Only the last token of
every sequence is projected unless input logprobs are requested; the vocab-parallel
product is gathered over the tensor ranks; padding columns are sliced off; optional
final soft-cap.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch
from torch import nn

from .. import ops
from ..parallel import state as ps


@dataclass
class LogitsProcessorOutput:
    next_token_logits: torch.Tensor | None = None          # [B, V]
    hidden_states: torch.Tensor | None = None
    next_token_logprobs: torch.Tensor | None = None        # [B]
    next_token_top_logprobs_val: list | None = None
    next_token_top_logprobs_idx: list | None = None
    next_token_token_ids_logprobs_val: list | None = None
    next_token_token_ids_logprobs_idx: list | None = None
    input_token_logprobs: torch.Tensor | None = None       # flat over requested input positions
    input_top_logprobs_val: list | None = None
    input_top_logprobs_idx: list | None = None
    input_token_ids_logprobs_val: list | None = None
    input_token_ids_logprobs_idx: list | None = None
    routed_experts: Any = None
    extras: dict = field(default_factory=dict)


class LogitsProcessor(nn.Module):
    def __init__(self, vocab_size: int, soft_cap: float | None = None, skip_all_gather: bool = False):
        super().__init__()
        self.vocab_size = vocab_size
        self.soft_cap = soft_cap
        self.skip_all_gather = skip_all_gather

    def _project(self, hidden: torch.Tensor, lm_head, local_only: bool = False, fused_gather: bool = True) -> torch.Tensor:
        """`fused_gather`: the peer-store gather returns a view of one symmetric buffer that the next such call
        overwrites, so only the step's next-token logits (consumed before the next step) go through it."""
        logits = ops.linear(hidden, lm_head.weight)
        if local_only:
            # this rank's vocab shard (padding columns included); the sampler reduces across ranks
            return logits
        if lm_head.tp_size > 1 and not self.skip_all_gather:
            comm = ps.get_state().fused_comm
            if fused_gather and comm is not None and comm.supports_logits_gather(logits):
                logits = comm.logits_gather(logits)
            else:
                logits = ps.all_gather(logits, dim=-1)
        logits = logits[:, : self.vocab_size]
        if self.soft_cap:
            logits = self.soft_cap * torch.tanh(logits.float() / self.soft_cap)
        return logits

    @staticmethod
    def _owned(t: torch.Tensor) -> torch.Tensor:
        """Hidden states handed to a consumer outside this step (embeddings, draft models) must not alias the
        fused-communication context's gather buffer, which the next fused call on any model overwrites."""
        comm = ps.get_state().fused_comm
        if comm is not None and t.is_cuda and \
                t.untyped_storage().data_ptr() == comm.gathered.tensor.untyped_storage().data_ptr():
            return t.clone()
        return t

    def forward(self, hidden_states: torch.Tensor, lm_head, forward_batch) -> LogitsProcessorOutput:
        fb = forward_batch
        if fb.forward_mode.is_decode() or fb.last_token_indices is None:
            last = hidden_states
        else:
            last = hidden_states[fb.last_token_indices]
        local_only = bool(fb.extras.get("skip_logits_gather")) and lm_head.tp_size > 1 and not self.soft_cap
        # speculative flows keep several logits tensors alive inside one step: they stay off the shared gather buffer
        plain_step = getattr(fb, "spec_info", None) is None and fb.capture_hidden_mode == 0
        out = LogitsProcessorOutput(next_token_logits=self._project(last, lm_head, local_only, fused_gather=plain_step))
        if local_only:
            out.extras["vocab_shard"] = (lm_head.vocab_start, self.vocab_size)
        if fb.capture_hidden_mode == 1:
            out.hidden_states = self._owned(last)
        elif fb.capture_hidden_mode == 2:
            out.hidden_states = self._owned(hidden_states)
        if fb.return_logprob and fb.forward_mode.is_extend() and fb.extend_logprob_start_lens_cpu is not None:
            self._input_logprobs(hidden_states, lm_head, fb, out)
        return out

    def _input_logprobs(self, hidden_states, lm_head, fb, out: LogitsProcessorOutput):
        """Log-probabilities of the prompt tokens from `logprob_start_len` on: row i of a
        sequence predicts token i+1, so the rows `[start, len-1)` are scored against the
        input ids shifted by one."""
        rows, targets, counts = [], [], []
        o = 0
        ids = fb.input_ids
        for b, (ext, start) in enumerate(zip(fb.extend_seq_lens_cpu.tolist(),
                                             fb.extend_logprob_start_lens_cpu.tolist())):
            n = max(ext - 1 - start, 0)
            if n:
                rows.append(torch.arange(o + start, o + start + n, device=hidden_states.device))
                targets.append(ids[o + start + 1: o + start + 1 + n])
            counts.append(n)
            o += ext
        out.extras["input_logprob_counts"] = counts
        if not rows:
            out.input_token_logprobs = torch.empty(0, device=hidden_states.device)
            return
        rows_t = torch.cat(rows)
        tgt = torch.cat(targets).long()
        logits = self._project(hidden_states[rows_t], lm_head, fused_gather=False).float()
        lp = torch.log_softmax(logits, dim=-1)
        out.input_token_logprobs = lp.gather(1, tgt.unsqueeze(1)).squeeze(1)
        out.extras["input_logprobs_full"] = lp
