"""CUDA-graph capture / replay of the decode step.

The reference avoids per-step compilation by padding batches to shape buckets and
pre-compiling one XLA executable per bucket (`python/sgl_jax/srt/model_executor/
compilation_manager.py:69-128`), and asserts zero recompiles at serving time.  The B200
equivalent: one captured CUDA graph per batch-size bucket holding the whole decode step
(future-token resolve, page-table delta scatter, all layers, LM head, sampling,
future-map store) in two variants: greedy (argmax, reduced across tensor ranks as (max, index) pairs) and
sampled (temperature / top-k / top-p / min-p through the sampling kernel on the gathered logits).  A step copies its few integers into the graph's static input buffers
and replays; nothing is captured after warm-up (`graph_recaptures` stays 0 and is
reported to clients as `cache_miss_count`).
"""

from __future__ import annotations

import bisect
import logging

import numpy as np
import torch

from ..managers.schedule_batch import ForwardMode, ModelWorkerBatch
from .forward_batch_info import ForwardBatch

logger = logging.getLogger(__name__)

DEFAULT_BS_BUCKETS = [1, 2, 4, 8, 12, 16, 24, 32, 40, 48, 56, 64, 80, 96, 112, 128, 160, 192, 224, 256]
MAX_PAGE_DELTAS = 1024


class CudaGraphRunner:
    def __init__(self, runner):
        self.runner = runner
        sa = runner.server_args
        max_bs = sa.cuda_graph_max_bs or min(runner.max_running_requests, 256)
        buckets = sa.precompile_bs_paddings or DEFAULT_BS_BUCKETS
        self.buckets = sorted({b for b in buckets if b <= max_bs} | {min(max_bs, max(buckets))})
        self.max_bs = self.buckets[-1]
        dev = runner.device
        self.pad_row = runner.req_to_token_pool.size   # all-zero page-table row -> dummy page 0
        n = self.max_bs
        # static inputs: ids | positions | out_cache_loc | req_pool | seq_lens | future_slots | delta rows,pos,ids |
        # sampling: top_ks | seeds | sample positions | temperatures | top_ps | min_ps (the last three are float bits)
        self.samp0 = 6 * n + 3 * MAX_PAGE_DELTAS
        self.buf = torch.zeros(self.samp0 + 6 * n, dtype=torch.int32, device=dev)
        self.host = torch.zeros(self.samp0 + 6 * n, dtype=torch.int32, pin_memory=True)
        # keys: batch-size bucket (greedy step) or (bucket, "sampled")
        self.graphs: dict = {}
        self.outputs: dict = {}
        self.seed_rng = np.random.default_rng(int(getattr(sa, "random_seed", 0) or 0) + 7919)
        # sampled steps need the full-vocabulary logits on every tensor rank: under tensor parallelism they are
        # captured when the peer-store gather of the fused-communication context can serve the bucket (its
        # symmetric result buffer is allocated by the eager warm-up step, never inside a capture); without that
        # context tensor-parallel engines sample eagerly
        from ..parallel import state as ps
        comm = ps.get_state().fused_comm
        self.sample_in_graph = ps.tp_size() == 1 or comm is not None
        self.sample_max_bs = self.max_bs if ps.tp_size() == 1 or comm is None else min(self.max_bs, comm.LOGITS_GATHER_ROWS)
        self.pool = None
        self.stream = torch.cuda.Stream(device=dev)
        self.copy_event: torch.cuda.Event | None = None
        self.enabled = True
        self.kernels_per_graph = 0
        self.swa_page_table: torch.Tensor | None = None
        if not sa.disable_precompile:
            self.capture_all()

    # ------------------------------------------------------------------
    def _views(self, bs: int):
        n = self.max_bs
        b = self.buf
        return dict(input_ids=b[0:bs], positions=b[n:n + bs], out_cache_loc=b[2 * n:2 * n + bs],
                    req_pool_indices=b[3 * n:3 * n + bs], seq_lens=b[4 * n:4 * n + bs],
                    future_slots=b[5 * n:5 * n + bs],
                    d_rows=b[6 * n:6 * n + MAX_PAGE_DELTAS],
                    d_pos=b[6 * n + MAX_PAGE_DELTAS:6 * n + 2 * MAX_PAGE_DELTAS],
                    d_ids=b[6 * n + 2 * MAX_PAGE_DELTAS:6 * n + 3 * MAX_PAGE_DELTAS],
                    top_ks=b[self.samp0:self.samp0 + bs], seeds=b[self.samp0 + n:self.samp0 + n + bs],
                    sample_pos=b[self.samp0 + 2 * n:self.samp0 + 2 * n + bs],
                    temperatures=b[self.samp0 + 3 * n:self.samp0 + 3 * n + bs].view(torch.float32),
                    top_ps=b[self.samp0 + 4 * n:self.samp0 + 4 * n + bs].view(torch.float32),
                    min_ps=b[self.samp0 + 5 * n:self.samp0 + 5 * n + bs].view(torch.float32))

    def _step(self, bs: int, sampled: bool = False) -> torch.Tensor:
        r = self.runner
        v = self._views(bs)
        from ..ops import native
        # page-table deltas: unused entries point at the padding row, which stays zero
        native.page_table_scatter(r.req_to_token_pool.page_table, v["d_rows"], v["d_pos"], v["d_ids"])
        ids = native.resolve_future(v["input_ids"], r.future_token_ids_map)
        fb = ForwardBatch(
            forward_mode=ForwardMode.DECODE, batch_size=bs, num_tokens=bs, input_ids=ids, positions=v["positions"],
            out_cache_loc=v["out_cache_loc"], req_pool_indices=v["req_pool_indices"], seq_lens=v["seq_lens"],
            page_table=r.req_to_token_pool.page_table, page_size=r.page_size,
            max_seq_len=r.model_config.context_len, token_to_kv_pool=r.token_to_kv_pool,
            attn_backend=r.attn_backend, in_graph=True)
        if getattr(r, "recurrent_pool", None) is not None:
            # hybrid linear-attention models: states are updated in place in slot row + 1; padding rows use the
            # scratch slot 0 (their page-table row index is one past the last request row)
            rows = v["req_pool_indices"].long()
            fb.extras["recurrent_pool"] = r.recurrent_pool
            fb.extras["recurrent_slots"] = torch.where(rows < self.pad_row, rows + 1, torch.zeros_like(rows))
        pool = r.token_to_kv_pool
        if hasattr(pool, "swa_pool"):
            # hybrid sliding-window models: the window layers' page table is derived from the (just updated)
            # full one through the full -> window slot mapping, rows of this batch only
            P = r.page_size
            pt = r.req_to_token_pool.page_table
            rows = v["req_pool_indices"].long()
            if self.swa_page_table is None:
                self.swa_page_table = torch.zeros_like(pt)
            self.swa_page_table[rows] = (pool.full_to_swa_index_mapping[pt[rows].long() * P] // P).to(pt.dtype)
            fb.extras["swa_page_table"] = self.swa_page_table
        from ..parallel import state as ps
        comm = ps.get_state().fused_comm
        if comm is not None and not sampled:
            fb.extras["skip_logits_gather"] = True
        r.select_residual_dataflow(fb)
        out = r.model(ids, fb)
        if sampled:
            # unseeded requests: fresh per-row seeds arrive with the step's inputs; every tensor rank holds the
            # same gathered logits and the same seeds, so all ranks draw the same tokens
            tok = native.sample_filtered(out.next_token_logits, v["temperatures"], v["top_ks"], v["top_ps"],
                                         v["min_ps"], v["seeds"], v["sample_pos"], request_seeded=False)
        elif "vocab_shard" in out.extras:
            start, vocab = out.extras["vocab_shard"]
            tok = comm.argmax_gather(out.next_token_logits, start, vocab)
        else:
            tok = native.argmax(out.next_token_logits)
        r.future_token_ids_map[v["future_slots"].long()] = tok
        return tok

    def capture_all(self):
        r = self.runner
        logger.info("capturing CUDA graphs for decode batch sizes %s", self.buckets)
        # make the padded inputs valid before the warm-up runs
        self._fill_padding(0, self.max_bs)
        with torch.inference_mode():
            for sampled in ((False, True) if self.sample_in_graph else (False,)):
                for bs in reversed(self.buckets):
                    if sampled and bs > self.sample_max_bs:
                        continue
                    torch.cuda.synchronize()
                    s = self.stream
                    s.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(s):
                        for _ in range(2):
                            self._step(bs, sampled)     # warm-up: lazy inits (function attributes, scratch) happen here
                    torch.cuda.current_stream().wait_stream(s)
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    from ..ops import native
                    n0 = native.launch_count
                    with torch.cuda.graph(g, pool=self.pool, stream=s):
                        out = self._step(bs, sampled)
                    if not sampled:
                        # kernels of this library inside one replay (torch's own small ops not counted)
                        self.kernels_per_graph = native.launch_count - n0
                    self.pool = self.pool or g.pool()
                    key = (bs, "sampled") if sampled else bs
                    self.graphs[key] = g
                    self.outputs[key] = out
        torch.cuda.synchronize()

    def _fill_padding(self, lo: int, hi: int):
        n = self.max_bs
        h = self.host.numpy()
        h[0 * n + lo:0 * n + hi] = 0
        h[1 * n + lo:1 * n + hi] = 0
        h[2 * n + lo:2 * n + hi] = 0
        h[3 * n + lo:3 * n + hi] = self.pad_row
        h[4 * n + lo:4 * n + hi] = 1
        h[5 * n + lo:5 * n + hi] = 0
        h[6 * n:6 * n + MAX_PAGE_DELTAS] = self.pad_row
        h[6 * n + MAX_PAGE_DELTAS:self.samp0] = 0
        self._fill_sampling_padding(lo, hi)
        self.buf.copy_(self.host, non_blocking=False)

    def _fill_sampling_padding(self, lo: int, hi: int):
        """Padding rows sample greedily (top_k 1): the cheapest path of the kernel."""
        n, s0 = self.max_bs, self.samp0
        h = self.host.numpy()
        f = h.view(np.float32)
        h[s0 + lo:s0 + hi] = 1
        h[s0 + n + lo:s0 + n + hi] = 0
        h[s0 + 2 * n + lo:s0 + 2 * n + hi] = 0
        f[s0 + 3 * n + lo:s0 + 3 * n + hi] = 1.0
        f[s0 + 4 * n + lo:s0 + 4 * n + hi] = 1.0
        f[s0 + 5 * n + lo:s0 + 5 * n + hi] = 0.0

    # ------------------------------------------------------------------
    def can_run(self, batch: ModelWorkerBatch) -> bool:
        si = batch.sampling_info
        return (self.enabled and batch.forward_mode.is_decode() and len(batch.req_pool_indices) <= self.max_bs
                and not batch.return_logprob and batch.capture_hidden_mode == 0 and batch.spec_info is None
                and (si is None or (si.linear_penalty is None and si.vocab_mask is None and si.logit_bias is None
                                    and getattr(si, "penalties", None) is None
                                    and (si.is_all_greedy or self._can_sample_in_graph(si, len(batch.req_pool_indices)))))
                and (batch.page_delta_rows is None or len(batch.page_delta_rows) <= MAX_PAGE_DELTAS)
                and not any(batch.lora_ids or []) and getattr(batch, "mrope_positions", None) is None)

    def _can_sample_in_graph(self, si, bs: int) -> bool:
        """Sampled steps run in a graph when no request carries its own seed (seeded and deterministic runs keep
        the reference's hash, which the eager sampler applies) and the logits are fp32 / bf16 on this device."""
        sa = self.runner.server_args
        return (self.sample_in_graph and si.sampling_seeds is None
                and self.buckets[bisect.bisect_left(self.buckets, bs)] <= self.sample_max_bs
                and not getattr(sa, "enable_deterministic_sampling", False) and si.positions is not None)

    def replay(self, batch: ModelWorkerBatch):
        r = self.runner
        bs = len(batch.req_pool_indices)
        bucket = self.buckets[bisect.bisect_left(self.buckets, bs)]
        si = batch.sampling_info
        sampled = si is not None and not si.is_all_greedy
        key = (bucket, "sampled") if sampled else bucket
        if key not in self.graphs:
            # capture on demand (only when precompile was disabled); counted like a jit cache miss
            r.graph_recaptures += 1
            self._capture_one(bucket, sampled)
        n = self.max_bs
        if self.copy_event is not None:
            self.copy_event.synchronize()     # the previous step's H2D has consumed the pinned buffer
        h = self.host.numpy()
        h[0:bs] = batch.input_ids
        h[n:n + bs] = batch.positions
        h[2 * n:2 * n + bs] = batch.out_cache_loc
        h[3 * n:3 * n + bs] = batch.req_pool_indices
        h[4 * n:4 * n + bs] = batch.seq_lens
        h[5 * n:5 * n + bs] = batch.future_slots if batch.future_slots is not None else 0
        if bucket > bs:
            h[0:n][bs:bucket] = 0
            h[n:2 * n][bs:bucket] = 0
            h[2 * n:3 * n][bs:bucket] = 0
            h[3 * n:4 * n][bs:bucket] = self.pad_row
            h[4 * n:5 * n][bs:bucket] = 1
            h[5 * n:6 * n][bs:bucket] = 0
        nd = 0 if batch.page_delta_rows is None else len(batch.page_delta_rows)
        d0 = 6 * n
        h[d0:d0 + MAX_PAGE_DELTAS] = self.pad_row
        h[d0 + MAX_PAGE_DELTAS:d0 + 3 * MAX_PAGE_DELTAS] = 0
        if nd:
            h[d0:d0 + nd] = batch.page_delta_rows
            h[d0 + MAX_PAGE_DELTAS:d0 + MAX_PAGE_DELTAS + nd] = batch.page_delta_pos
            h[d0 + 2 * MAX_PAGE_DELTAS:d0 + 2 * MAX_PAGE_DELTAS + nd] = batch.page_delta_ids
        if sampled:
            s0 = self.samp0
            f = h.view(np.float32)
            h[s0:s0 + bs] = si.top_ks
            h[s0 + n:s0 + n + bs] = self.seed_rng.integers(0, 2 ** 31 - 1, size=bs, dtype=np.int32)
            h[s0 + 2 * n:s0 + 2 * n + bs] = si.positions
            f[s0 + 3 * n:s0 + 3 * n + bs] = si.temperatures
            f[s0 + 4 * n:s0 + 4 * n + bs] = si.top_ps
            f[s0 + 5 * n:s0 + 5 * n + bs] = si.min_ps
            if bucket > bs:
                self._fill_sampling_padding(bs, bucket)
        self.buf.copy_(self.host, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.copy_event = ev
        self.graphs[key].replay()
        r.graph_replays += 1
        r.h2d_bytes_total += self.host.numel() * 4
        return None, self.outputs[key][:bs], None

    def _capture_one(self, bs: int, sampled: bool = False):
        with torch.inference_mode():
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            s = self.stream
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._step(bs, sampled)
            torch.cuda.current_stream().wait_stream(s)
            with torch.cuda.graph(g, pool=self.pool, stream=s):
                out = self._step(bs, sampled)
            self.pool = self.pool or g.pool()
            key = (bs, "sampled") if sampled else bs
            self.graphs[key] = g
            self.outputs[key] = out
