"""Token sampling.

Pipeline of the reference (`python/sgl_jax/srt/layers/sampler.py:166-458`): additive
penalties -> logit bias -> grammar bitmask -> greedy argmax when every row is greedy,
else temperature / top-k / top-p / min-p filtering and a multinomial draw.  Rows with a
`sampling_seed` use the hash-Gumbel draw that depends only on (seed, position, column),
so the result does not depend on which other requests share the batch.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
from torch import nn

from .. import ops
from ..ops import reference


@dataclass
class SamplingMetadata:
    """Device-side sampling controls for one batch."""
    temperatures: torch.Tensor
    top_ks: torch.Tensor
    top_ps: torch.Tensor
    min_ps: torch.Tensor
    is_all_greedy: bool
    need_filter: bool
    sampling_seeds: torch.Tensor | None = None
    positions: torch.Tensor | None = None
    linear_penalty: torch.Tensor | None = None
    logit_bias: torch.Tensor | None = None
    vocab_mask: torch.Tensor | None = None
    return_logprob: bool = False
    top_logprobs_nums: list | None = None
    token_ids_logprobs: list | None = None

    @classmethod
    def from_worker_batch(cls, batch, device) -> "SamplingMetadata":
        si = batch.sampling_info

        def t(a, dt=None):
            if a is None:
                return None
            x = torch.from_numpy(np.ascontiguousarray(a))
            return x.to(device, non_blocking=True) if dt is None else x.to(device=device, dtype=dt, non_blocking=True)

        if si.is_all_greedy and si.linear_penalty is None and si.vocab_mask is None and si.logit_bias is None \
                and not batch.return_logprob:
            # nothing to upload for the common greedy case
            return cls(None, None, None, None, True, False)
        return cls(
            temperatures=t(si.temperatures), top_ks=t(si.top_ks), top_ps=t(si.top_ps), min_ps=t(si.min_ps),
            is_all_greedy=si.is_all_greedy,
            need_filter=si.need_top_k_sampling or si.need_top_p_sampling or si.need_min_p_sampling,
            sampling_seeds=t(si.sampling_seeds), positions=t(si.positions),
            linear_penalty=t(si.linear_penalty), logit_bias=t(si.logit_bias), vocab_mask=t(si.vocab_mask),
            return_logprob=batch.return_logprob, top_logprobs_nums=batch.top_logprobs_nums,
            token_ids_logprobs=batch.token_ids_logprobs,
        )


class Sampler(nn.Module):
    def __init__(self, rng_seed: int = 42, use_sort_for_toppk_minp: bool = False,
                 enable_deterministic: bool = False, enable_nan_detection: bool = False):
        super().__init__()
        self.rng_seed = rng_seed
        self.enable_deterministic = enable_deterministic
        self.enable_nan_detection = enable_nan_detection
        self._gen: torch.Generator | None = None
        self.step = 0

    def _generator(self, device) -> torch.Generator:
        if self._gen is None or self._gen.device != device:
            self._gen = torch.Generator(device=device)
            self._gen.manual_seed(self.rng_seed)
        return self._gen

    def forward(self, logits_output, meta: SamplingMetadata) -> torch.Tensor:
        """Returns int32 `[B]` next-token ids and fills logprob fields of `logits_output`."""
        logits = logits_output.next_token_logits
        if meta.linear_penalty is not None:
            logits = logits.float() + meta.linear_penalty
        if meta.logit_bias is not None:
            logits = logits.float() + meta.logit_bias
        if meta.vocab_mask is not None:
            logits = reference.apply_token_bitmask(logits.float(), meta.vocab_mask)
        if self.enable_nan_detection and torch.isnan(logits).any():
            logits = torch.where(torch.isnan(logits), torch.full_like(logits, -1e5), logits)
        if meta.is_all_greedy:
            ids = ops.argmax(logits)
            probs_for_lp = None
        else:
            if ops.use_native_sampling(logits):
                ids = self._sample_native(logits, meta)
            else:
                ids = self._sample_reference(logits, meta)
            ids = ids.to(torch.int32)
        self.step += 1
        if meta.return_logprob:
            self.compute_logprobs(logits, ids, logits_output, meta)
        return ids

    def _seeds_and_positions(self, meta: SamplingMetadata, B: int, device):
        """Per-row (seed, position) of the hashed Gumbel draw: the request's own seed, a fixed one under
        `enable_deterministic`, otherwise fresh seeds from this sampler's generator."""
        if meta.sampling_seeds is not None:
            seeds = meta.sampling_seeds
        elif self.enable_deterministic:
            seeds = torch.full((B,), 42, dtype=torch.int32, device=device)
        else:
            seeds = torch.randint(0, 2 ** 31 - 1, (B,), dtype=torch.int32, device=device,
                                  generator=self._generator(device))
        positions = meta.positions if meta.positions is not None else \
            torch.full((B,), self.step, dtype=torch.int32, device=device)
        return seeds, positions

    def _sample_native(self, logits, meta: SamplingMetadata) -> torch.Tensor:
        """One kernel: temperature, top-k / top-p / min-p (sort-free radix select) and the hashed Gumbel-max
        draw; rows with `top_k <= 1` come back as the argmax."""
        seeds, positions = self._seeds_and_positions(meta, logits.shape[0], logits.device)
        if logits.stride(-1) != 1:
            logits = logits.contiguous()
        seeded = meta.sampling_seeds is not None or self.enable_deterministic
        return ops._native().sample_filtered(logits, meta.temperatures, meta.top_ks, meta.top_ps, meta.min_ps, seeds,
                                             positions, request_seeded=seeded)

    def _sample_reference(self, logits, meta: SamplingMetadata) -> torch.Tensor:
        lf = logits.float()
        if meta.need_filter:
            probs = reference.top_k_top_p_min_p_probs(lf, meta.temperatures, meta.top_ks, meta.top_ps, meta.min_ps)
        else:
            probs = torch.softmax(lf / meta.temperatures.view(-1, 1).clamp_min(1e-6), dim=-1)
        if meta.sampling_seeds is not None or self.enable_deterministic:
            seeds, positions = self._seeds_and_positions(meta, probs.shape[0], probs.device)
            ids = reference.multinomial_with_seed(probs, seeds, positions)
        else:
            ids = torch.multinomial(probs, 1, generator=self._generator(probs.device)).squeeze(1)
        greedy_rows = meta.top_ks <= 1
        if bool(greedy_rows.any()):
            ids = torch.where(greedy_rows, torch.argmax(lf, dim=-1), ids)
        return ids

    @staticmethod
    def compute_logprobs(logits, ids, out, meta: SamplingMetadata):
        lp = torch.log_softmax(logits.float(), dim=-1)
        out.next_token_logprobs = lp.gather(1, ids.long().unsqueeze(1)).squeeze(1)
        if meta.top_logprobs_nums and any(n > 0 for n in meta.top_logprobs_nums):
            kmax = max(meta.top_logprobs_nums)
            tv, ti = lp.topk(kmax, dim=-1)
            tv, ti = tv.tolist(), ti.tolist()
            out.next_token_top_logprobs_val = [tv[i][:n] for i, n in enumerate(meta.top_logprobs_nums)]
            out.next_token_top_logprobs_idx = [ti[i][:n] for i, n in enumerate(meta.top_logprobs_nums)]
        if meta.token_ids_logprobs and any(t for t in meta.token_ids_logprobs):
            vals, idxs = [], []
            for i, toks in enumerate(meta.token_ids_logprobs):
                if toks:
                    vals.append(lp[i, torch.as_tensor(toks, device=lp.device)].tolist())
                    idxs.append(list(toks))
                else:
                    vals.append([])
                    idxs.append([])
            out.next_token_token_ids_logprobs_val = vals
            out.next_token_token_ids_logprobs_idx = idxs
