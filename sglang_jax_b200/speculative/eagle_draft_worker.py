"""The draft side of EAGLE / EAGLE-3 / NEXTN / STANDALONE speculative decoding.

Conventions (`L` = number of tokens of a request whose KV is in the cache, `t_L` = its last
sampled token, which has no KV yet):

* the draft input at cache position `i` is the pair (token `i+1`, target hidden state `i`),
  so the draft cache of a request is exactly as long as the target cache and the two
  share slot indices;
* depth-`d` tree tokens are fed at draft position `L + d - 1`; the `k` branches of draft
  step `s` occupy the tail slots `(s-1)*k .. s*k-1` of the step's reservation and see each
  other through an ancestor mask, which makes the branch caches exact for any page size;
* after verification the accepted tokens are re-run through the draft with the target's
  true hidden states (`draft_extend_after_verify`), which overwrites the speculative draft
  entries of those positions and yields the first level of the next tree.

Reference: `python/sgl_jax/srt/speculative/eagle_draft_worker.py`,
`multi_layer_draft_worker.py`, `draft_extend_fused.py`.
"""

from __future__ import annotations

import numpy as np
import torch

from ..managers.schedule_batch import ForwardMode
from .base_worker import BaseDraftWorker, BaseSpecWorker, SpecInput
from .eagle_util import select_top_k_branches


class EagleDraftWorker(BaseDraftWorker):
    def __init__(self, server_args, target_worker, algo, owner: BaseSpecWorker):
        super().__init__(server_args, target_worker, algo, owner.topk)
        self.owner = owner
        self.num_steps = owner.num_steps
        self.uses_hidden = bool(getattr(self.model, "is_eagle_draft", False))

    def decorate_spec(self, spec: SpecInput, step: int | None) -> SpecInput:
        """Hook for subclasses: `step` is the draft step of a tree-growing forward, None for
        the passes that fill the draft cache."""
        return spec

    # ------------------------------------------------------------------ prefill
    @torch.inference_mode()
    def draft_extend_for_prefill(self, mwb, next_ids: torch.Tensor, hidden: torch.Tensor | None,
                                 chunk_next: np.ndarray):
        """Run the draft over a prefill batch.  `mwb` is the target's worker batch,
        `next_ids [B]` the tokens it sampled, `hidden [T, *]` the target hidden states of the
        extend tokens, `chunk_next [B]` the prompt token following a non-final chunk (-1 for
        rows that really sampled)."""
        B = len(mwb.req_pool_indices)
        ids = torch.from_numpy(np.asarray(mwb.input_ids)).to(self.device).long()
        ext = np.asarray(mwb.extend_seq_lens)
        cu = np.concatenate([[0], np.cumsum(ext)])
        last = torch.from_numpy(cu[1:] - 1).to(self.device).long()
        shifted = torch.roll(ids, -1)
        nxt = next_ids.long()
        cn = torch.from_numpy(chunk_next.astype(np.int64)).to(self.device)
        shifted[last] = torch.where(cn >= 0, cn, nxt)
        spec = self.decorate_spec(
            SpecInput(input_ids=shifted.int(), hidden_states=hidden if self.uses_hidden else None), None)
        batch = self.owner.make_batch(ForwardMode.DRAFT_EXTEND, np.asarray(mwb.req_pool_indices),
                                      np.asarray(mwb.seq_lens), np.asarray(mwb.out_cache_loc),
                                      np.asarray(mwb.extend_prefix_lens), ext, spec, 1, len(ids),
                                      positions=np.asarray(mwb.positions))
        out, _, _ = self.runner.forward(batch, skip_sample=True)
        rows = torch.from_numpy(np.asarray(mwb.req_pool_indices)).to(self.device).long()
        self.store_first_level(rows, out.next_token_logits, out.hidden_states, torch.where(cn >= 0, cn, nxt))

    # ------------------------------------------------------------------ decode: multi-step draft
    @torch.inference_mode()
    def draft(self, rows_np: np.ndarray, L: np.ndarray, tail_slots: np.ndarray):
        """Grow the candidate tree for every request.

        `tail_slots [B, alloc_len]` are the KV slots reserved for this step.  Returns
        `(cand_tokens, cand_scores, cand_parent)` over all candidates, `[B, C]`, with
        `cand_parent` holding parent node ids."""
        k, S = self.topk, self.num_steps
        B = len(rows_np)
        dev = self.device
        rows = torch.from_numpy(rows_np.astype(np.int64)).to(dev)
        # level 1 comes from the cached state
        tok_levels = [self.state_topk_index[rows]]                  # [B, k]
        score_levels = [self.state_topk_p[rows]]
        parent_levels = [torch.zeros(B, k, dtype=torch.long, device=dev)]
        branch_tok = tok_levels[0]
        branch_score = score_levels[0]
        branch_node = torch.arange(1, k + 1, device=dev).expand(B, -1)
        hidden = self.state_hidden[rows].unsqueeze(1).expand(B, k, -1) if self.uses_hidden else None
        anc = torch.zeros(B, k, max((S - 1) * k, 1), dtype=torch.bool, device=dev)
        L_t = torch.from_numpy(L.astype(np.int64)).to(dev)
        for s in range(1, S):
            # feed the k branches of depth s; they occupy tail slots (s-1)*k .. s*k-1
            lo, hi = (s - 1) * k, s * k
            ar = torch.arange(k, device=dev)
            anc[:, ar, lo + ar] = True
            pos = (L_t + (s - 1)).view(B, 1).expand(B, k).reshape(-1)
            spec = SpecInput(input_ids=branch_tok.reshape(-1).int(), positions=pos.int(), all_logits=True,
                             hidden_states=hidden.reshape(B * k, -1) if hidden is not None else None,
                             custom_mask=None if k == 1 else anc[:, :, :hi].contiguous())
            spec = self.decorate_spec(spec, s)
            batch = self.owner.make_batch(
                ForwardMode.DRAFT_EXTEND, rows_np, L + hi, tail_slots[:, lo:hi].reshape(-1),
                L + lo, np.full(B, k, np.int32), spec, 2, B * k)
            out, _, _ = self.runner.forward(batch, skip_sample=True)
            probs = torch.softmax(out.next_token_logits.float(), dim=-1).view(B, k, -1)
            c_tok, c_score, c_branch, sel = select_top_k_branches(s, k, branch_score, probs, 0)
            c_tok = self.map_ids(c_tok)
            tok_levels.append(c_tok)
            score_levels.append(c_score)
            parent_levels.append(branch_node.gather(1, c_branch))
            base = 1 + k + (s - 1) * k * k
            src_branch = c_branch.gather(1, sel)                    # parent branch of every new branch
            branch_tok = c_tok.gather(1, sel)
            branch_score = c_score.gather(1, sel)
            branch_node = base + sel
            if hidden is not None:
                h = out.hidden_states.view(B, k, -1)
                hidden = h.gather(1, src_branch.unsqueeze(-1).expand(-1, -1, h.shape[-1]))
            anc = anc.gather(1, src_branch.unsqueeze(-1).expand(-1, -1, anc.shape[-1]))
        return torch.cat(tok_levels, 1), torch.cat(score_levels, 1), torch.cat(parent_levels, 1)

    # ------------------------------------------------------------------ decode: after verify
    @torch.inference_mode()
    def draft_extend_after_verify(self, rows_np: np.ndarray, L: np.ndarray, accept_np: np.ndarray,
                                  tail_slots: np.ndarray, new_tokens: torch.Tensor, hidden: torch.Tensor | None,
                                  bonus: torch.Tensor):
        """`new_tokens` (flat, ragged: accepted draft tokens then the bonus token per request)
        are fed at positions `L .. L+a` with the target's hidden states `hidden` (flat, same
        order)."""
        B = len(rows_np)
        ext = (accept_np + 1).astype(np.int32)
        total = int(ext.sum())
        positions = np.concatenate([np.arange(l, l + e, dtype=np.int32) for l, e in zip(L, ext)])
        loc = np.concatenate([tail_slots[b, :ext[b]] for b in range(B)])
        spec = self.decorate_spec(
            SpecInput(input_ids=new_tokens.int(), hidden_states=hidden if self.uses_hidden else None), None)
        batch = self.owner.make_batch(ForwardMode.DRAFT_EXTEND, rows_np, L + ext, loc, L, ext, spec, 1, total,
                                      positions=positions)
        out, _, _ = self.runner.forward(batch, skip_sample=True)
        rows = torch.from_numpy(rows_np.astype(np.int64)).to(self.device)
        self.store_first_level(rows, out.next_token_logits, out.hidden_states, bonus)
