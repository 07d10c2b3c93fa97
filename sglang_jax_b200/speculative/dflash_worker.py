"""DFLASH speculative decoding: a block-diffusion drafter proposes `block_size - 1` tokens in
ONE forward, the target verifies the block as a chain.

Per step and request (`L` cached tokens, anchor `t_L`):
  1. reserve `block_size` slots behind `L`;
  2. draft forward over `[t_L, MASK, ..., MASK]` at positions `L..L+block-1`, bidirectional
     inside the block, attending to the context KV that was materialised from target
     features; position `j >= 1` yields draft token `d_j`;
  3. target TARGET_VERIFY over `[t_L, d_1, ...]` (causal); greedy / stochastic chain accept;
  4. the draft KV of the accepted positions is re-materialised from the target features of
     the verify pass (the block's own provisional entries are overwritten).

Reference: `python/sgl_jax/srt/speculative/dflash_worker.py`.
"""

from __future__ import annotations

import logging

import numpy as np
import torch

from ..managers.schedule_batch import ForwardMode, ScheduleBatch
from ..managers.tp_worker import GenerationBatchResult
from ..model_executor.forward_batch_info import ForwardBatch
from .base_worker import BaseDraftWorker, BaseSpecWorker, SpecInput
from .eagle_util import tree_speculative_sampling_target_only, verify_tree_greedy
from .eagle_worker import EAGLEWorker
from .spec_info import SpeculativeAlgorithm

logger = logging.getLogger(__name__)


class DFlashWorker(EAGLEWorker):
    def __init__(self, server_args, target_worker):
        BaseSpecWorker.__init__(self, server_args, target_worker, SpeculativeAlgorithm.DFLASH)
        self.draft_worker = BaseDraftWorker(server_args, target_worker, SpeculativeAlgorithm.DFLASH, 1)
        dm = self.draft_worker.model
        embed, head = self.target_runner.model.get_embed_and_head()
        dm.set_embed_and_head(embed, head)
        self.block_size = int(dm.block_size)
        if server_args.speculative_num_draft_tokens and server_args.speculative_num_draft_tokens > 1:
            self.block_size = int(server_args.speculative_num_draft_tokens)
        self.num_draft_tokens = self.block_size
        self.num_steps = self.block_size - 1
        self.topk = 1
        self.alloc_len = self.block_size
        self.mask_token_id = dm.mask_token_id
        self.uses_aux = True
        self.sim_acc = None
        layer_ids = dm.target_layer_ids or list(range(self.target_runner.model_config.num_hidden_layers))[-dm.num_context_features:]
        self.target_runner.model.set_eagle3_layers_to_capture(layer_ids)
        logger.info("speculative decoding: DFLASH, block=%d, target feature layers=%s", self.block_size, layer_ids)

    # ------------------------------------------------------------------ prefill
    def _materialize(self, rows_np, seq_lens, loc_np, pre, ext, positions_np, features):
        dw = self.draft_worker
        spec = SpecInput()
        batch = self.make_batch(ForwardMode.DRAFT_EXTEND, rows_np, seq_lens, loc_np, pre, ext, spec, 0,
                                len(loc_np), positions=positions_np)
        fb = ForwardBatch.init_new(batch, dw.runner)
        dw.model.materialize_kv(features, fb.positions, fb.out_cache_loc, fb)

    def _prefill(self, batch: ScheduleBatch) -> GenerationBatchResult:
        mwb = batch.get_model_worker_batch()
        self.target_worker.spec_broadcast("spec_prefill", (mwb, None, False))
        return self.prefill_core(mwb, None, False)

    @torch.inference_mode()
    def prefill_core(self, mwb, chunk_next=None, want_hidden: bool = False) -> GenerationBatchResult:
        mwb.capture_hidden_mode = 2
        res = self.target_worker.forward_batch_generation(mwb, broadcast=False)
        out = res.logits_output
        feats = self._target_hidden(out)
        self._materialize(np.asarray(mwb.req_pool_indices), np.asarray(mwb.seq_lens), np.asarray(mwb.out_cache_loc),
                          np.asarray(mwb.extend_prefix_lens), np.asarray(mwb.extend_seq_lens),
                          np.asarray(mwb.positions), feats)
        rows = torch.from_numpy(np.asarray(mwb.req_pool_indices)).to(self.device).long()
        self.draft_worker.state_verified[rows] = res.next_token_ids.long()
        out.hidden_states = None
        return res

    # ------------------------------------------------------------------ decode
    @torch.inference_mode()
    def decode_core(self, rows_np, L, tail, deltas, sinfo) -> GenerationBatchResult:
        dw = self.draft_worker
        dev = self.device
        self.pending_deltas = deltas
        B, n = len(rows_np), self.block_size
        rows = torch.from_numpy(rows_np.astype(np.int64)).to(dev)
        anchor = dw.state_verified[rows]
        L_t = torch.from_numpy(L.astype(np.int64)).to(dev)
        pos = (L_t.view(B, 1) + torch.arange(n, device=dev).view(1, n)).reshape(-1)

        # ---- one draft forward proposes the whole block
        block = torch.full((B, n), self.mask_token_id, dtype=torch.long, device=dev)
        block[:, 0] = anchor
        full = torch.ones(B, n, n, dtype=torch.bool, device=dev)
        spec = SpecInput(input_ids=block.reshape(-1).int(), positions=pos.int(), all_logits=True, custom_mask=full)
        db = self.make_batch(ForwardMode.DRAFT_EXTEND, rows_np, L + n, tail[:, :n].reshape(-1), L,
                             np.full(B, n, np.int32), spec, 0, B * n)
        dout, _, _ = dw.runner.forward(db, skip_sample=True)
        proposal = dout.next_token_logits.view(B, n, -1).argmax(dim=-1)
        tokens = torch.cat([anchor.view(B, 1), proposal[:, 1:]], dim=1)
        parent = (torch.arange(n, device=dev) - 1).expand(B, -1).contiguous()

        # ---- verify the chain
        vspec = SpecInput(input_ids=tokens.reshape(-1).int(), positions=pos.int(), all_logits=True)
        vb = self.make_batch(ForwardMode.TARGET_VERIFY, rows_np, L + n, tail[:, :n].reshape(-1), L,
                             np.full(B, n, np.int32), vspec, 2, B * n)
        out, _, _ = self.target_runner.forward(vb, skip_sample=True)
        logits = out.next_token_logits.view(B, n, -1)
        if sinfo.is_all_greedy:
            accept, path, bonus = verify_tree_greedy(tokens, parent, logits.argmax(dim=-1), n - 1)
        else:
            accept, path, bonus = self._stochastic_verify(tokens, parent, logits, sinfo, n - 1)
        acc_np = accept.cpu().numpy().astype(np.int64)
        tok_np = tokens.cpu().numpy()
        bonus_np = bonus.cpu().numpy()
        out_tokens = [[int(t) for t in tok_np[b, 1:acc_np[b] + 1]] + [int(bonus_np[b])] for b in range(B)]

        # ---- draft KV of the accepted positions comes from the target features
        ext = (acc_np + 1).astype(np.int32)
        flat = torch.from_numpy(np.concatenate([b * n + np.arange(ext[b]) for b in range(B)])).to(dev)
        feats = self._target_hidden(out)[flat]
        positions = np.concatenate([np.arange(l, l + e, dtype=np.int32) for l, e in zip(L, ext)])
        loc = np.concatenate([tail[b, :ext[b]] for b in range(B)])
        self._materialize(rows_np, L + ext, loc, L, ext, positions, feats)
        dw.state_verified[rows] = bonus.long()

        res = GenerationBatchResult(None, None, bid=vb.bid)
        res.spec_tokens = out_tokens
        res.accept_lens = acc_np
        res.alloc_ends = (L + self.alloc_len).astype(np.int64)
        return res
