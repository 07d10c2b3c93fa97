"""Device-side view of one step's batch.

Counterpart of the reference's `ForwardBatch`
(`python/sgl_jax/srt/model_executor/forward_batch_info.py:148-495`).  All integer
metadata of a step is packed into ONE pinned host buffer and moved with ONE
host→device copy; the fields below are views into that device buffer.  The
page table is not part of the upload: it lives on the device permanently and the
batch only carries the entries that changed (`page_delta_*`).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch

from ..managers.schedule_batch import ForwardMode, ModelWorkerBatch


class CaptureHiddenMode:
    NULL = 0
    LAST = 1
    FULL = 2


class _PinnedRing:
    """A few pinned int32 staging buffers used round-robin so an async H2D copy of
    step n is never overwritten by the packing of step n+1."""

    def __init__(self, n_bufs: int, capacity: int, device: str):
        self.device = device
        self.use_pinned = device != "cpu" and torch.cuda.is_available()
        self.bufs = [torch.empty(capacity, dtype=torch.int32, pin_memory=self.use_pinned)
                     for _ in range(n_bufs)]
        self.events = [None] * n_bufs
        self.i = 0

    def next(self, need: int) -> tuple[torch.Tensor, int]:
        self.i = (self.i + 1) % len(self.bufs)
        if self.bufs[self.i].numel() < need:
            self.bufs[self.i] = torch.empty(max(need, 2 * self.bufs[self.i].numel()),
                                            dtype=torch.int32, pin_memory=self.use_pinned)
        ev = self.events[self.i]
        if ev is not None:
            ev.synchronize()
        return self.bufs[self.i], self.i

    def mark(self, idx: int):
        if self.use_pinned:
            ev = torch.cuda.Event()
            ev.record()
            self.events[idx] = ev


@dataclass
class ForwardBatch:
    forward_mode: ForwardMode
    batch_size: int
    num_tokens: int
    input_ids: torch.Tensor
    positions: torch.Tensor
    out_cache_loc: torch.Tensor
    req_pool_indices: torch.Tensor
    seq_lens: torch.Tensor
    page_table: torch.Tensor
    page_size: int
    # extend only
    extend_prefix_lens: torch.Tensor | None = None
    extend_seq_lens: torch.Tensor | None = None
    cu_q_lens: torch.Tensor | None = None          # [B+1]
    max_extend_len: int = 0
    max_seq_len: int = 0
    # host copies (reference path, logprob slicing)
    seq_lens_cpu: np.ndarray | None = None
    extend_prefix_lens_cpu: np.ndarray | None = None
    extend_seq_lens_cpu: np.ndarray | None = None
    # rows of the hidden states that produce logits: last token of every sequence
    last_token_indices: torch.Tensor | None = None
    return_logprob: bool = False
    extend_logprob_start_lens_cpu: np.ndarray | None = None
    capture_hidden_mode: int = CaptureHiddenMode.NULL
    token_to_kv_pool: Any = None
    attn_backend: Any = None
    lora_ids: list | None = None
    spec_info: Any = None
    num_decode_in_mixed: int = 0
    h2d_bytes: int = 0
    # set while a CUDA graph is being captured / replayed
    in_graph: bool = False
    extras: dict = field(default_factory=dict)

    @classmethod
    def init_new(cls, batch: ModelWorkerBatch, runner) -> "ForwardBatch":
        mode = batch.forward_mode
        T = len(batch.input_ids)
        B = len(batch.req_pool_indices)
        nd = 0 if batch.page_delta_rows is None else len(batch.page_delta_rows)
        is_ext = mode.is_extend()
        # layout: input_ids | positions | out_cache_loc | req_pool | seq_lens | [prefix | extend | cu_q(B+1)] | delta x3
        sizes = [T, T, T, B, B] + ([B, B, B + 1] if is_ext else []) + [nd, nd, nd]
        total = sum(sizes)
        ring: _PinnedRing = runner.staging
        host, slot = ring.next(total)
        h = host.numpy()
        o = 0

        def put(arr, n):
            nonlocal o
            if n:
                h[o:o + n] = arr
            o += n
            return (o - n, o)

        spans = [put(batch.input_ids, T), put(batch.positions, T), put(batch.out_cache_loc, T),
                 put(batch.req_pool_indices, B), put(batch.seq_lens, B)]
        if is_ext:
            cu = np.zeros(B + 1, np.int32)
            np.cumsum(batch.extend_seq_lens, out=cu[1:])
            spans += [put(batch.extend_prefix_lens, B), put(batch.extend_seq_lens, B), put(cu, B + 1)]
        spans += [put(batch.page_delta_rows, nd), put(batch.page_delta_pos, nd), put(batch.page_delta_ids, nd)]
        dev = host[:total].to(runner.device, non_blocking=True)
        ring.mark(slot)
        v = [dev[a:b] for a, b in spans]
        if nd:
            d_rows, d_pos, d_ids = v[-3], v[-2], v[-1]
            runner.req_to_token_pool.page_table[d_rows.long(), d_pos.long()] = d_ids
        fb = cls(
            forward_mode=mode, batch_size=B, num_tokens=T,
            input_ids=v[0], positions=v[1], out_cache_loc=v[2], req_pool_indices=v[3], seq_lens=v[4],
            page_table=runner.req_to_token_pool.page_table, page_size=runner.page_size,
            seq_lens_cpu=np.asarray(batch.seq_lens),
            max_seq_len=int(batch.seq_lens.max()) if B else 0,
            return_logprob=batch.return_logprob,
            capture_hidden_mode=batch.capture_hidden_mode,
            token_to_kv_pool=runner.token_to_kv_pool, attn_backend=runner.attn_backend,
            lora_ids=batch.lora_ids, spec_info=batch.spec_info,
            num_decode_in_mixed=batch.num_decode_in_mixed,
            h2d_bytes=total * 4,
        )
        if getattr(runner, "recurrent_pool", None) is not None:
            fb.extras["recurrent_pool"] = runner.recurrent_pool
            if getattr(batch, "recurrent_tracks", None):
                fb.extras["recurrent_tracks"] = {int(i): (int(k), int(slot)) for i, k, slot in batch.recurrent_tracks}
        if getattr(batch, "deepstack_embeds", None) is not None:
            fb.extras["deepstack"] = batch.deepstack_embeds.to(runner.device, runner.dtype)
        if getattr(batch, "mrope_positions", None) is not None:
            fb.extras["mrope_positions"] = torch.from_numpy(np.ascontiguousarray(batch.mrope_positions)).to(
                runner.device, non_blocking=True)
        pool = runner.token_to_kv_pool
        if hasattr(pool, "swa_pool") and B:
            # sliding-window layers live in their own (smaller) pool: translate the rows' pages
            P = runner.page_size
            pt = runner.req_to_token_pool.page_table
            rows_l = fb.req_pool_indices.long()
            swa_pt = torch.zeros_like(pt)
            swa_pt[rows_l] = (pool.full_to_swa_index_mapping[(pt[rows_l].long() * P)] // P).to(pt.dtype)
            fb.extras["swa_page_table"] = swa_pt
        if is_ext:
            fb.extend_prefix_lens, fb.extend_seq_lens, fb.cu_q_lens = v[5], v[6], v[7]
            fb.extend_prefix_lens_cpu = np.asarray(batch.extend_prefix_lens)
            fb.extend_seq_lens_cpu = np.asarray(batch.extend_seq_lens)
            fb.max_extend_len = int(batch.extend_seq_lens.max()) if B else 0
            fb.last_token_indices = (fb.cu_q_lens[1:] - 1).long()
            fb.extend_logprob_start_lens_cpu = batch.extend_logprob_start_lens
        return fb
