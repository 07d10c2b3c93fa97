"""Consumes forward results: appends tokens, checks finish conditions, keeps logprob
records, moves finished requests' KV into the prefix cache and streams outputs to the
detokenizer.

Reference: `python/sgl_jax/srt/managers/scheduler_output_processor_mixin.py`
(prefill :140, decode :373, `add_input_logprob_return_values` :596,
`stream_output_generation` :776-993).
"""

from __future__ import annotations

import time

import numpy as np

from ..global_config import global_config
from .io_struct import BatchEmbeddingOut, BatchTokenIDOut
from .schedule_batch import FINISH_ABORT, Req, ScheduleBatch


class SchedulerOutputProcessorMixin:
    # ------------------------------------------------------------------ prefill
    def process_batch_result_prefill(self, batch: ScheduleBatch, result):
        ids = self.tp_worker.resolve(result).tolist() if result.next_token_ids is not None else []
        self._collect_routed_experts(batch, result)
        lo = result.logits_output
        n_prefill = len(batch.reqs) - batch.num_decode_in_mixed
        lp_val = lo.next_token_logprobs.tolist() if (lo is not None and lo.next_token_logprobs is not None) else None
        in_lp = None
        if lo is not None and lo.input_token_logprobs is not None:
            in_lp = lo.input_token_logprobs.tolist()
            in_counts = lo.extras.get("input_logprob_counts")
        in_off = 0
        for i, req in enumerate(batch.reqs):
            if req.finished() or req.is_retracted:
                # aborted while its prefill was in flight (or retracted): nothing to record
                if in_lp is not None:
                    in_off += in_counts[i]
                continue
            is_decode_row = i >= n_prefill
            if not is_decode_row and req.is_chunked > 0:
                # a non-final chunk: KV is written, no token is produced
                req.is_chunked -= 1
                if in_lp is not None:
                    self._add_input_logprobs(req, in_lp[in_off:in_off + in_counts[i]], batch, i, last_chunk=False)
                    in_off += in_counts[i]
                continue
            tok = int(ids[i])
            req.output_ids.append(tok)
            if req.first_token_time is None:
                req.first_token_time = time.perf_counter()
            if req.return_logprob:
                if in_lp is not None and not is_decode_row:
                    self._add_input_logprobs(req, in_lp[in_off:in_off + in_counts[i]], batch, i, last_chunk=True)
                self._add_output_logprobs(req, lo, i, tok, lp_val)
            if in_lp is not None:
                in_off += in_counts[i]
            if req.return_hidden_states and lo is not None and lo.hidden_states is not None:
                req.hidden_states.append(lo.hidden_states[i].float().cpu().tolist())
            if req.grammar is not None:
                req.grammar.accept_token(tok)
            req.check_finished()
            if req.finished():
                self._finish_req(req)
            elif not is_decode_row:
                # publish the prompt in the prefix cache so followers can share it
                self.tree_cache.cache_unfinished_req(req)
        self.stream_output(batch.reqs, batch.return_logprob)

    def _collect_routed_experts(self, batch: ScheduleBatch, result):
        """Hand every request that asked for them the routed expert ids of the tokens this step computed for it
        (`[tokens, layers, top_k]` per step; tokens served from the prefix cache were not computed)."""
        snap = getattr(result, "routed_experts", None)
        if snap is None:
            return
        from ..layers.routed_experts_capturer import RoutedExpertsCapturer
        if batch.forward_mode.is_extend() and batch.extend_lens:
            lens = [int(x) for x in batch.extend_lens]
        else:
            lens = [1] * len(batch.reqs)
        spans, o = [], 0
        for n in lens:
            spans.append((o, n))
            o += n
        for req, arr in zip(batch.reqs, RoutedExpertsCapturer.per_request(snap[0], snap[1], spans)):
            if req.return_routed_experts and not req.is_retracted and not req.finished():
                req.routed_experts.extend(arr.tolist())

    # ------------------------------------------------------------------ decode
    def process_batch_result_decode(self, batch: ScheduleBatch, result):
        ids = self.tp_worker.resolve(result).tolist()
        self._collect_routed_experts(batch, result)
        lo = result.logits_output
        lp_val = lo.next_token_logprobs.tolist() if (lo is not None and lo.next_token_logprobs is not None) else None
        self.num_generated_tokens += len(batch.reqs)
        for i, req in enumerate(batch.reqs):
            if req.finished() or req.is_retracted:
                # finished one step earlier (overlap mode runs one step ahead): its KV was
                # already handed to the cache / freed together with the request
                continue
            tok = int(ids[i])
            req.output_ids.append(tok)
            if req.return_logprob:
                self._add_output_logprobs(req, lo, i, tok, lp_val)
            if req.return_hidden_states and lo is not None and lo.hidden_states is not None:
                req.hidden_states.append(lo.hidden_states[i].float().cpu().tolist())
            if req.grammar is not None:
                req.grammar.accept_token(tok)
            req.check_finished()
            if req.finished():
                self._finish_req(req)
        self.stream_output(batch.reqs, batch.return_logprob)
        self.forward_ct_decode += 1
        if self.forward_ct_decode % self.server_args.decode_log_interval == 0:
            self.log_decode_stats(batch)

    def process_batch_result_spec_decode(self, batch: ScheduleBatch, result):
        """A speculative step yields 1..num_draft_tokens tokens per request (reference
        `scheduler_output_processor_mixin.py`, `accept_lens` / strided `next_token_ids`).
        Tokens are appended one at a time so a stop condition inside the accepted run cuts
        it; then the unused part of the step's KV reservation is returned."""
        ps = self.page_size
        alloc = self.token_to_kv_pool_allocator
        for i, req in enumerate(batch.reqs):
            if req.finished() or req.is_retracted:
                continue
            L = req.kv_committed_len
            m = 0
            for tok in result.spec_tokens[i]:
                req.output_ids.append(int(tok))
                m += 1
                req.check_finished()
                if req.finished():
                    break
            req.spec_verify_ct += 1
            req.spec_accepted_tokens += m - 1
            self.num_generated_tokens += m
            self.spec_num_total_accepted_tokens += m
            self.spec_num_total_forward_ct += 1
            req.kv_committed_len = L + m
            keep = (req.kv_committed_len + ps - 1) // ps * ps
            end = int(result.alloc_ends[i])
            if end > keep:
                alloc.free(self.req_to_token_pool.read(req.req_pool_idx, end)[keep:].copy(), dp_rank=batch.dp_rank)
            req.kv_allocated_len = req.kv_committed_len
            if req.finished():
                self._finish_req(req)
        self.stream_output(batch.reqs, batch.return_logprob)
        self.forward_ct_decode += 1
        if self.forward_ct_decode % self.server_args.decode_log_interval == 0:
            self.log_decode_stats(batch)

    def process_batch_result_embedding(self, batch: ScheduleBatch, embeddings):
        emb = embeddings.float().cpu().tolist()
        rids, outs, ptoks, reasons = [], [], [], []
        for i, req in enumerate(batch.reqs):
            if req.is_chunked > 0:
                req.is_chunked -= 1
                continue
            req.finished_reason = req.finished_reason or _EmbeddingDone()
            self._finish_req(req, insert=True)
            rids.append(req.rid)
            outs.append(emb[i])
            ptoks.append(len(req.origin_input_ids))
            reasons.append({"type": "stop"})
        if rids:
            self.send_to_detokenizer(BatchEmbeddingOut(rids, reasons, outs, ptoks))

    # ------------------------------------------------------------------ helpers
    def _finish_req(self, req: Req, insert: bool = True):
        req.finished_time = time.perf_counter()
        if getattr(self, "disagg_mode", "null") == "prefill" and self.disagg_prefill_hold(req):
            return      # the KV stays until the decode engine has pulled it
        if getattr(self, "disagg_mode", "null") == "decode" and getattr(req, "pd_time_stats", None) is not None:
            from ..disaggregation import req_time_stats
            req_time_stats.mark(self, req, "finished", final=True)
        if req.req_pool_idx is not None:
            self.tree_cache.cache_finished_req(req, is_insert=insert and not isinstance(req.finished_reason, FINISH_ABORT))
            self.req_to_token_pool.free(req.req_pool_idx)
            req.req_pool_idx = None
        if req.grammar is not None and hasattr(req.grammar, "finished"):
            req.grammar.finished = True

    def _add_output_logprobs(self, req: Req, lo, i: int, tok: int, lp_val):
        if lp_val is not None:
            req.output_token_logprobs_val.append(lp_val[i])
            req.output_token_logprobs_idx.append(tok)
        if req.top_logprobs_num > 0 and lo.next_token_top_logprobs_val is not None:
            req.output_top_logprobs_val.append(lo.next_token_top_logprobs_val[i])
            req.output_top_logprobs_idx.append(lo.next_token_top_logprobs_idx[i])
        if req.token_ids_logprob and lo.next_token_token_ids_logprobs_val is not None:
            req.output_token_ids_logprobs_val.append(lo.next_token_token_ids_logprobs_val[i])
            req.output_token_ids_logprobs_idx.append(lo.next_token_token_ids_logprobs_idx[i])

    def _add_input_logprobs(self, req: Req, vals: list, batch: ScheduleBatch, i: int, last_chunk: bool):
        """Accumulate prompt-token logprobs over chunks.  The first prompt token has no
        predecessor, so its logprob is reported as None."""
        if req.return_output_logprob_only:
            return
        if req.input_token_logprobs_val is None:
            req.input_token_logprobs_val = []
            req.input_token_logprobs_idx = []
            start = max(req.logprob_start_len, 0) if req.logprob_start_len >= 0 else len(req.origin_input_ids) - 1
            if start == 0:
                req.input_token_logprobs_val.append(None)
                req.input_token_logprobs_idx.append(req.origin_input_ids[0])
            req._input_lp_next = start + 1
        n = len(vals)
        nxt = req._input_lp_next
        req.input_token_logprobs_val.extend(vals)
        req.input_token_logprobs_idx.extend(req.fill_ids[nxt:nxt + n] if nxt + n <= len(req.fill_ids)
                                            else (req.origin_input_ids + req.output_ids)[nxt:nxt + n])
        req._input_lp_next = nxt + n
        if req.top_logprobs_num > 0 and req.input_top_logprobs_val is None:
            req.input_top_logprobs_val, req.input_top_logprobs_idx = [], []

    # ------------------------------------------------------------------ streaming
    def stream_output(self, reqs: list[Req], return_logprob: bool = False):
        """Send new tokens of finished requests and of streaming requests whose turn it is
        (every `stream_interval` tokens, at least every 50; the first token always)."""
        if self.is_embedding:
            return
        out = BatchTokenIDOut([], [], [], [], [], [], [], [], [], [], [], [])
        force = global_config.default_force_stream_interval
        for req in reqs:
            if req.is_retracted or req.is_chunked > 0 and not req.finished():
                continue
            if getattr(req, "_finished_output_sent", False):
                continue
            if req.finished():
                req._finished_output_sent = True
                should = True
            elif req.stream:
                interval = req.sampling_params.stream_interval or self.stream_interval
                n = len(req.output_ids)
                should = n > 0 and (n == 1 or n % interval == 0 or n % force == 0)
            else:
                should = False   # non-streaming requests report once, when they finish
            if not should:
                continue
            if req.finished_len is not None and not req.sampling_params.no_stop_trim:
                out_ids = req.output_ids[: req.finished_len]
            else:
                out_ids = req.output_ids
            decode_ids, read_offset = req.init_incremental_detokenize()
            out.rids.append(req.rid)
            out.finished_reasons.append(req.finished_reason.to_json() if req.finished_reason else None)
            out.decoded_texts.append(req.decoded_text)
            out.decode_ids.append(decode_ids[req.send_decode_id_offset:])
            req.send_decode_id_offset = len(decode_ids)
            out.read_offsets.append(read_offset)
            if self.server_args.stream_output and not req.finished():
                out.output_ids.append(out_ids[req.send_token_offset:])
                req.send_token_offset = len(out_ids)
            else:
                out.output_ids.append(list(out_ids))
            out.skip_special_tokens.append(req.sampling_params.skip_special_tokens)
            out.spaces_between_special_tokens.append(req.sampling_params.spaces_between_special_tokens)
            out.no_stop_trim.append(req.sampling_params.no_stop_trim)
            out.prompt_tokens.append(len(req.origin_input_ids))
            out.completion_tokens.append(len(out_ids))
            out.cached_tokens.append(req.cached_tokens)
            if getattr(self, "section_rank", None) is not None:
                out.dp_ranks = (out.dp_ranks or []) + [self.section_rank]
            if return_logprob:
                first = not req.input_logprob_sent
                if req.return_logprob and first and req.input_token_logprobs_val is not None:
                    out.input_token_logprobs_val.append(req.input_token_logprobs_val)
                    out.input_token_logprobs_idx.append(req.input_token_logprobs_idx)
                    out.input_top_logprobs_val.append(req.input_top_logprobs_val or [])
                    out.input_top_logprobs_idx.append(req.input_top_logprobs_idx or [])
                    out.input_token_ids_logprobs_val.append(req.input_token_ids_logprobs_val or [])
                    out.input_token_ids_logprobs_idx.append(req.input_token_ids_logprobs_idx or [])
                    req.input_logprob_sent = True
                else:
                    for lst in (out.input_token_logprobs_val, out.input_token_logprobs_idx, out.input_top_logprobs_val,
                                out.input_top_logprobs_idx, out.input_token_ids_logprobs_val,
                                out.input_token_ids_logprobs_idx):
                        lst.append([])
                s = req.send_output_token_logprobs_offset
                out.output_token_logprobs_val.append(req.output_token_logprobs_val[s:])
                out.output_token_logprobs_idx.append(req.output_token_logprobs_idx[s:])
                out.output_top_logprobs_val.append(req.output_top_logprobs_val[s:])
                out.output_top_logprobs_idx.append(req.output_top_logprobs_idx[s:])
                out.output_token_ids_logprobs_val.append(req.output_token_ids_logprobs_val[s:])
                out.output_token_ids_logprobs_idx.append(req.output_token_ids_logprobs_idx[s:])
                req.send_output_token_logprobs_offset = len(req.output_token_logprobs_val)
            if req.return_hidden_states:
                if out.output_hidden_states is None:
                    out.output_hidden_states = []
                out.output_hidden_states.append(req.hidden_states)
            if req.return_routed_experts:
                if out.output_routed_experts is None:
                    out.output_routed_experts = []
                out.output_routed_experts.append(req.routed_experts)
            if self.spec_algorithm is not None:
                if out.spec_verify_ct is None:
                    out.spec_verify_ct = []
                out.spec_verify_ct.append(req.spec_verify_ct)
        if out.rids:
            out.cache_miss_count = self.graph_recapture_count()
            self.send_to_detokenizer(out)


class _EmbeddingDone:
    is_error = False

    def to_json(self):
        return {"type": "stop"}
