"""Incremental detokenisation.

Reference: `python/sgl_jax/srt/managers/detokenizer_manager.py` (`DetokenizerManager` :51,
`handle_batch_token_id_out` :133, `LimitedCapacityDict` :316, `run_detokenizer_process` :329).
Each request keeps a *surrogate* window of already-emitted ids so that a new id is decoded in
context (multi-byte characters, leading spaces); text is only released once it no longer ends
in an incomplete UTF-8 sequence; stop strings are trimmed from the tail.
"""

from __future__ import annotations

import dataclasses
import logging
import os
import signal
from collections import OrderedDict

from ..global_config import global_config
from .io_struct import BatchEmbeddingOut, BatchStrOut, BatchTokenIDOut

logger = logging.getLogger(__name__)


class LimitedCapacityDict(OrderedDict):
    def __init__(self, capacity: int, *a, **k):
        super().__init__(*a, **k)
        self.capacity = capacity

    def __setitem__(self, key, value):
        if len(self) >= self.capacity and key not in self:
            self.popitem(last=False)
        super().__setitem__(key, value)


@dataclasses.dataclass
class DecodeStatus:
    decoded_text: str
    decode_ids: list[int]
    surr_offset: int
    read_offset: int
    sent_offset: int = 0


class DetokenizerManager:
    def __init__(self, server_args, port_args=None, recv=None, send=None, tokenizer=None):
        self.server_args = server_args
        self.recv = recv
        self.send = send
        if recv is None and port_args is not None:
            import zmq
            from .communication import get_zmq_socket
            ctx = zmq.Context(2)
            self.recv = get_zmq_socket(ctx, zmq.PULL, port_args.detokenizer_ipc_name, True)
            self.send = get_zmq_socket(ctx, zmq.PUSH, port_args.tokenizer_ipc_name, False)
        self.tokenizer = tokenizer
        if tokenizer is None and not server_args.skip_tokenizer_init:
            from ..utils.hf_transformers_utils import get_tokenizer
            self.tokenizer = get_tokenizer(server_args.tokenizer_path, server_args.tokenizer_mode,
                                           server_args.trust_remote_code, server_args.revision,
                                           server_args.tokenizer_backend)
        self.decode_status: LimitedCapacityDict = LimitedCapacityDict(global_config.detokenizer_max_states)

    def trim_matched_stop(self, text: str, finished_reason: dict | None, no_stop_trim: bool) -> str:
        if no_stop_trim or not finished_reason:
            return text
        matched = finished_reason.get("matched")
        if isinstance(matched, str) and matched:
            pos = text.find(matched)
            return text[:pos] if pos != -1 else text
        return text

    def handle_batch_embedding_out(self, recv: BatchEmbeddingOut):
        return recv

    def handle_batch_token_id_out(self, recv: BatchTokenIDOut) -> BatchStrOut:
        bs = len(recv.rids)
        if self.tokenizer is None:
            strs = [""] * bs
        else:
            read_ids, surr_ids = [], []
            for i in range(bs):
                rid = recv.rids[i]
                st = self.decode_status.get(rid)
                if st is None:
                    st = DecodeStatus(recv.decoded_texts[i], list(recv.decode_ids[i]), 0, recv.read_offsets[i])
                    self.decode_status[rid] = st
                else:
                    st.decode_ids.extend(recv.decode_ids[i])
                read_ids.append(st.decode_ids[st.surr_offset:])
                surr_ids.append(st.decode_ids[st.surr_offset:st.read_offset])
            kw = dict(skip_special_tokens=recv.skip_special_tokens[0] if bs else True,
                      spaces_between_special_tokens=recv.spaces_between_special_tokens[0] if bs else True)
            surr_texts = self.tokenizer.batch_decode(surr_ids, **kw)
            read_texts = self.tokenizer.batch_decode(read_ids, **kw)
            strs = []
            for i in range(bs):
                rid = recv.rids[i]
                st = self.decode_status[rid]
                new_text = read_texts[i][len(surr_texts[i]):]
                if recv.finished_reasons[i] is None:
                    if len(new_text) > 0 and not new_text.endswith("�"):
                        st.decoded_text += new_text
                        st.surr_offset = st.read_offset
                        st.read_offset = len(st.decode_ids)
                        new_text = ""
                    else:
                        # keep the incomplete tail back
                        new_text = new_text[: _safe_len(new_text)]
                out = self.trim_matched_stop(st.decoded_text + new_text, recv.finished_reasons[i], recv.no_stop_trim[i])
                if self.server_args.stream_output and recv.finished_reasons[i] is None:
                    strs.append(out[st.sent_offset:])
                    st.sent_offset = len(out)
                else:
                    strs.append(out)
                if recv.finished_reasons[i] is not None:
                    self.decode_status.pop(rid, None)
        return BatchStrOut(
            rids=recv.rids, finished_reasons=recv.finished_reasons, output_strs=strs, output_ids=recv.output_ids,
            prompt_tokens=recv.prompt_tokens, completion_tokens=recv.completion_tokens,
            cached_tokens=recv.cached_tokens,
            input_token_logprobs_val=recv.input_token_logprobs_val, input_token_logprobs_idx=recv.input_token_logprobs_idx,
            output_token_logprobs_val=recv.output_token_logprobs_val, output_token_logprobs_idx=recv.output_token_logprobs_idx,
            input_top_logprobs_val=recv.input_top_logprobs_val, input_top_logprobs_idx=recv.input_top_logprobs_idx,
            output_top_logprobs_val=recv.output_top_logprobs_val, output_top_logprobs_idx=recv.output_top_logprobs_idx,
            input_token_ids_logprobs_val=recv.input_token_ids_logprobs_val,
            input_token_ids_logprobs_idx=recv.input_token_ids_logprobs_idx,
            output_token_ids_logprobs_val=recv.output_token_ids_logprobs_val,
            output_token_ids_logprobs_idx=recv.output_token_ids_logprobs_idx,
            output_hidden_states=recv.output_hidden_states, cache_miss_count=recv.cache_miss_count,
            output_routed_experts=recv.output_routed_experts, spec_verify_ct=recv.spec_verify_ct,
            dp_ranks=recv.dp_ranks)

    def handle(self, obj):
        if isinstance(obj, BatchTokenIDOut):
            return self.handle_batch_token_id_out(obj)
        return obj   # embeddings and control replies pass through

    def event_loop(self, stop_event=None):
        import queue as _q
        while stop_event is None or not stop_event.is_set():
            try:
                obj = self.recv.recv_pyobj(timeout=0.05) if hasattr(self.recv, "q") else self.recv.recv_pyobj()
            except _q.Empty:
                continue
            self.send.send_pyobj(self.handle(obj))


def _safe_len(text: str) -> int:
    n = len(text)
    while n > 0 and text[n - 1] == "�":
        n -= 1
    return n


def run_detokenizer_process(server_args, port_args):
    from ..utils.common import configure_logger, kill_itself_when_parent_died
    kill_itself_when_parent_died()
    configure_logger(server_args)
    try:
        DetokenizerManager(server_args, port_args).event_loop()
    except Exception:
        import traceback
        logger.error("DetokenizerManager hit an exception: %s", traceback.format_exc())
        os.kill(os.getppid(), signal.SIGQUIT)
