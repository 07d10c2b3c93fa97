"""Rank 0 -> follower ranks channel for the per-step batch.

The reference is single-controller (one process feeds every device), so it has no such hop inside a
node; across nodes node 0 mirrors its requests over ZMQ PUB/SUB
(`python/sgl_jax/srt/managers/scheduler.py:625-676,:1215-1257`).  Here there is one process per GPU and
the scheduler on tensor rank 0 ships every step's `ModelWorkerBatch` to the other ranks.  On one node
that goes through a shared-memory ring (`csrc/sched/sched_native.cpp: StepRing`): a plain decode / extend
step travels as one fixed-layout block of int32 (no pickling, no socket, no host collective), anything
richer (log-probabilities, adapters, speculative inputs, control messages) as a pickled blob through the
same ring, so ordering is preserved.  Across nodes the channel is a ZMQ PUB / SUB mirror (rank 0 publishes, the other
nodes subscribe; sequence numbers expose a dropped message), or `broadcast_object_list` when no address is given.

Failure detection: a follower that stops consuming fills the ring, and the producer's `send` raises after
`timeout_s`; a follower waits in bounded slices and gives up when the ring is closed.
"""

from __future__ import annotations

import os
import pickle
import uuid

import numpy as np

from . import state as ps

KIND_PICKLE = 0
KIND_BATCH = 1
KIND_PART = 2          # piece of a pickled message that does not fit one slot; KIND_PICKLE ends it

SLOT_BYTES = 1 << 20
SLOTS = 8

_HDR = 16              # int32 words of the fixed-layout header


def _plain(batch) -> bool:
    si = batch.sampling_info
    return (not batch.return_logprob and batch.top_logprobs_nums is None and batch.token_ids_logprobs is None
            and not batch.return_output_logprob_only and not any(batch.lora_ids or [])
            and batch.spec_info is None and batch.spec_algorithm is None and batch.input_embeds is None
            and batch.input_embeds_rows is None and batch.mrope_positions is None and batch.deepstack_embeds is None
            and not batch.recurrent_copies and not batch.recurrent_tracks and batch.extend_logprob_start_lens is None
            and batch.launch_done is None
            and (si is None or (si.linear_penalty is None and si.vocab_mask is None and si.logit_bias is None
                                and getattr(si, "penalties", None) is None)))


def encode_batch(batch) -> np.ndarray | None:
    """`ModelWorkerBatch` -> int32 block, or None when the batch carries more than a plain step's integers."""
    if not _plain(batch):
        return None
    B, T = len(batch.req_pool_indices), len(batch.input_ids)
    nd = 0 if batch.page_delta_rows is None else len(batch.page_delta_rows)
    ext = batch.extend_seq_lens is not None
    fut = batch.future_slots is not None
    si = batch.sampling_info
    seeds = si is not None and si.sampling_seeds is not None
    spos = si is not None and si.positions is not None
    flags = 0
    if si is not None:
        flags = 1 | (2 if si.is_all_greedy else 0) | (4 if si.need_top_p_sampling else 0) | \
            (8 if si.need_top_k_sampling else 0) | (16 if si.need_min_p_sampling else 0) | \
            (32 if seeds else 0) | (64 if spos else 0)
    parts = [np.array([batch.bid, int(batch.forward_mode.value), B, T, nd, int(ext), int(fut), flags,
                       batch.num_decode_in_mixed, batch.capture_hidden_mode, batch.real_bs, batch.dp_rank,
                       int(batch.lora_ids is not None), 0, 0, 0], np.int32)]

    def put(a, n):
        a = np.asarray(a)
        assert a.shape == (n,), (a.shape, n)
        parts.append(a.astype(np.int32, copy=False))

    put(batch.input_ids, T)
    put(batch.out_cache_loc, T)
    put(batch.positions, T)
    put(batch.req_pool_indices, B)
    put(batch.seq_lens, B)
    if ext:
        put(batch.extend_prefix_lens, B)
        put(batch.extend_seq_lens, B)
    if fut:
        put(batch.future_slots, B)
    if nd:
        put(batch.page_delta_rows, nd)
        put(batch.page_delta_pos, nd)
        put(batch.page_delta_ids, nd)
    if si is not None:
        for f in (si.temperatures, si.top_ps, si.min_ps):
            parts.append(np.asarray(f, np.float32).view(np.int32))
        put(si.top_ks, B)
        if seeds:
            put(si.sampling_seeds, B)
        if spos:
            put(si.positions, B)
    return np.concatenate(parts)


def decode_batch(a: np.ndarray):
    from ..managers.schedule_batch import ForwardMode, ModelWorkerBatch, ModelWorkerSamplingInfo
    bid, mode, B, T, nd, ext, fut, flags, ndm, chm, real_bs, dp_rank, has_lora = (int(x) for x in a[:13])
    o = _HDR

    def take(n):
        nonlocal o
        v = a[o:o + n]
        o += n
        return v

    input_ids, out_cache_loc, positions = take(T), take(T), take(T)
    rows, seq_lens = take(B), take(B)
    pre = exl = None
    if ext:
        pre, exl = take(B), take(B)
    future = take(B).astype(np.int64) if fut else None
    d_rows = d_pos = d_ids = None
    if nd:
        d_rows, d_pos, d_ids = take(nd), take(nd), take(nd)
    si = None
    if flags & 1:
        t, p, m = (take(B).view(np.float32) for _ in range(3))
        k = take(B)
        seeds = take(B) if flags & 32 else None
        spos = take(B) if flags & 64 else None
        si = ModelWorkerSamplingInfo(temperatures=t, top_ps=p, top_ks=k, min_ps=m, sampling_seeds=seeds,
                                     is_all_greedy=bool(flags & 2), need_top_p_sampling=bool(flags & 4),
                                     need_top_k_sampling=bool(flags & 8), need_min_p_sampling=bool(flags & 16),
                                     positions=spos)
    return ModelWorkerBatch(bid=bid, forward_mode=ForwardMode(mode), input_ids=input_ids, req_pool_indices=rows,
                            seq_lens=seq_lens, out_cache_loc=out_cache_loc, positions=positions,
                            extend_prefix_lens=pre, extend_seq_lens=exl, page_delta_rows=d_rows,
                            page_delta_pos=d_pos, page_delta_ids=d_ids, sampling_info=si,
                            num_decode_in_mixed=ndm, capture_hidden_mode=chm, real_bs=real_bs, dp_rank=dp_rank,
                            lora_ids=[None] * B if has_lora else None, future_slots=future)


class StepChannel:
    """`send(obj)` on the group's first rank, `recv()` on the others."""

    def __init__(self, group, use_shm: bool = True, timeout_s: float = 120.0, pubsub_host: str | None = None):
        """`pubsub_host`: address of rank 0 that the other ranks can reach; selects the ZMQ PUB / SUB mirror (the
        reference's multi-node form, `managers/scheduler.py:625-676`: the leader publishes every step, follower
        nodes subscribe) instead of a host collective when the ranks do not share a node."""
        self.group = group
        self.is_root = group.rank == 0
        self.timeout_s = timeout_s
        self.ring = None
        self.pub = self.sub = None
        self.seq = 0
        self.sent_fixed = self.sent_pickled = 0
        if group.size <= 1:
            return
        ok = 0
        name = None
        if pubsub_host and not use_shm:
            self._init_pubsub(pubsub_host)
            return
        if use_shm:
            try:
                from ..mem_cache import _sched_native as sn
                name = ps.broadcast_object(f"/sglb_step_{os.getpid()}_{uuid.uuid4().hex[:8]}" if self.is_root else None,
                                           src=0, group=group)
                if self.is_root:
                    self.ring = sn.StepRing(name, SLOTS, SLOT_BYTES, group.size - 1)
                ps.barrier(group)
                if not self.is_root:
                    self.ring = sn.StepRing(name, SLOTS, SLOT_BYTES, group.size - 1, group.rank - 1)
                ok = 1
            except Exception:
                ok = 0
        # every rank must agree on the transport
        import torch
        import torch.distributed as dist
        t = torch.tensor([ok], dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group.cpu_group)
        if int(t.item()) == 0:
            self.ring = None

    def _init_pubsub(self, host: str):
        """Rank 0 binds a PUB socket, the others subscribe and then prove they receive: a PUB socket drops what is
        published before a subscriber has connected, so rank 0 publishes probes until every rank has seen one
        (checked through the host group), and only then the channel is open.  Messages carry a sequence number; a
        gap (dropped message: the subscriber fell behind its high-water mark) is an error, not silent skew."""
        import threading
        import zmq
        ctx = zmq.Context.instance()
        if self.is_root:
            self.pub = ctx.socket(zmq.PUB)
            self.pub.setsockopt(zmq.SNDHWM, 1 << 16)
            self.pub.setsockopt(zmq.LINGER, 2000)
            port = self.pub.bind_to_random_port("tcp://*")
            ps.broadcast_object(f"{host}:{port}", src=0, group=self.group)
            stop = threading.Event()

            def probe():
                while not stop.is_set():
                    self.pub.send_multipart([b"probe", b""])
                    stop.wait(0.01)
            t = threading.Thread(target=probe, daemon=True)
            t.start()
            ps.barrier(self.group)          # every subscriber has seen a probe
            stop.set()
            t.join()
        else:
            addr = ps.broadcast_object(None, src=0, group=self.group)
            self.sub = ctx.socket(zmq.SUB)
            self.sub.setsockopt(zmq.RCVHWM, 1 << 16)
            self.sub.setsockopt(zmq.SUBSCRIBE, b"")
            self.sub.connect(f"tcp://{addr}")
            if not self.sub.poll(int(self.timeout_s * 1000)):
                raise RuntimeError(f"no probe from rank 0 at {addr} within {self.timeout_s:.0f}s")
            ps.barrier(self.group)

    @property
    def transport(self) -> str:
        if self.pub is not None or self.sub is not None:
            return "zmq-pubsub"
        return "shm-ring" if self.ring is not None else ("none" if self.group.size <= 1 else "gloo-broadcast")

    # ------------------------------------------------------------------ root
    def send(self, obj) -> None:
        if self.group.size <= 1:
            return
        if self.pub is not None:
            from ..managers.schedule_batch import ModelWorkerBatch
            self.seq += 1
            head = self.seq.to_bytes(8, "little")
            ints = encode_batch(obj) if isinstance(obj, ModelWorkerBatch) else None
            if ints is not None:
                self.pub.send_multipart([b"batch", head, ints.tobytes()])
                self.sent_fixed += 1
            else:
                self.pub.send_multipart([b"pickle", head, pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)])
                self.sent_pickled += 1
            return
        if self.ring is None:
            ps.broadcast_object(obj, src=0, group=self.group)
            return
        from ..managers.schedule_batch import ModelWorkerBatch
        if isinstance(obj, ModelWorkerBatch):
            ints = encode_batch(obj)
            if ints is not None and ints.nbytes <= SLOT_BYTES:
                self._push(lambda: self.ring.push_ints(ints, KIND_BATCH, self.timeout_s))
                self.sent_fixed += 1
                return
        blob = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
        while len(blob) > SLOT_BYTES:
            head, blob = blob[:SLOT_BYTES], blob[SLOT_BYTES:]
            self._push(lambda: self.ring.push(head, KIND_PART, self.timeout_s))
        self._push(lambda: self.ring.push(blob, KIND_PICKLE, self.timeout_s))
        self.sent_pickled += 1

    def _push(self, fn):
        if not fn():
            who, lag = self.ring.slowest()
            raise RuntimeError(f"tensor rank {who + 1} stopped consuming step messages "
                               f"({lag} behind after {self.timeout_s:.0f}s)")

    def close(self):
        if self.ring is not None and self.is_root:
            self.ring.close()
        if self.pub is not None:
            self.pub.send_multipart([b"close", b""])
            self.pub.close()
            self.pub = None

    # ------------------------------------------------------------------ followers
    def recv(self, poll_s: float = 1.0, on_idle=None, block: bool = True):
        """Next message from rank 0.  Waits in `poll_s` slices (calling `on_idle()` between them);
        raises `EOFError` once rank 0 closed the channel.  `block=False` (ring transport only) returns `None`
        when no message has started to arrive within `poll_s`."""
        if self.sub is not None:
            while True:
                if not self.sub.poll(int(poll_s * 1000)):
                    if on_idle is not None:
                        on_idle()
                    if not block:
                        return None
                    continue
                frames = self.sub.recv_multipart()
                kind = frames[0]
                if kind == b"probe":
                    continue
                if kind == b"close":
                    raise EOFError("step channel closed by rank 0")
                seq = int.from_bytes(frames[1], "little")
                if seq != self.seq + 1:
                    raise RuntimeError(f"step channel lost messages {self.seq + 1}..{seq - 1} (subscriber fell behind)")
                self.seq = seq
                if kind == b"batch":
                    return decode_batch(np.frombuffer(frames[2], dtype=np.int32))
                return pickle.loads(frames[2])
        if self.ring is None:
            return ps.broadcast_object(None, src=0, group=self.group)
        parts = []
        while True:
            got = self.ring.pop(poll_s, True)
            if got is None:
                if self.ring.closed():
                    raise EOFError("step channel closed by rank 0")
                if not block and not parts:
                    return None
                if on_idle is not None:
                    on_idle()
                continue
            kind, payload = got
            if kind == KIND_BATCH:
                return decode_batch(payload)
            if kind == KIND_PART:
                parts.append(payload)
                continue
            return pickle.loads(b"".join(parts) + payload if parts else payload)
