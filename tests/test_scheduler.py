"""Scheduler behaviour against a mock worker (CPU): continuous batching, chunked prefill, prefix
reuse, retraction (incl. the forced-retract fault injection), abort, pause/continue, flush and
the KV leak invariant."""

import queue

import numpy as np
import pytest

from sglang_jax_b200.managers.io_struct import (AbortReq, ContinueGenerationReqInput, FlushCacheReqInput,
                                                PauseGenerationReqInput, TokenizedGenerateReqInput)
from sglang_jax_b200.managers.scheduler import Scheduler
from sglang_jax_b200.managers.tp_worker import MockModelWorker
from sglang_jax_b200.sampling.sampling_params import SamplingParams
from sglang_jax_b200.server_args import ServerArgs


def make(page_size=1, max_total=4096, overlap=False, max_running=64, chunk=4096, ctx=2048, **kw):
    sa = ServerArgs(model_path="mock", device="cpu", page_size=page_size, skip_tokenizer_init=True,
                    disable_overlap_schedule=not overlap, chunked_prefill_size=chunk, max_running_requests=max_running,
                    **kw)
    worker = MockModelWorker(sa, max_total_num_tokens=max_total, max_running_requests=max_running,
                             context_len=ctx, page_size=page_size)
    rq, sq = queue.Queue(), queue.Queue()
    return Scheduler(sa, None, tp_worker=worker, recv_queue=rq, send_queue=sq), rq, sq, worker


def req(rid, n_in, n_out=8, seed=None, ids=None, **sp):
    rng = np.random.RandomState(seed if seed is not None else hash(rid) % 1000)
    ids = ids if ids is not None else rng.randint(0, 1000, size=n_in).tolist()
    return TokenizedGenerateReqInput(rid=rid, input_ids=ids,
                                     sampling_params=SamplingParams(max_new_tokens=n_out, temperature=0.0,
                                                                    ignore_eos=True, **sp))


def run(s, sq, n_expected, max_steps=5000):
    done = {}
    step = s.step_overlap if s.enable_overlap else s.step_normal
    for _ in range(max_steps):
        step()
        while not sq.empty():
            o = sq.get()
            if not hasattr(o, "rids"):
                continue
            for rid, ids, fr in zip(o.rids, o.output_ids, o.finished_reasons):
                if fr is not None:
                    done[rid] = (ids, fr)
        if len(done) >= n_expected:
            break
    for _ in range(4):
        step()
    return done


@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("page_size", [1, 16])
def test_continuous_batching_and_leak_invariant(overlap, page_size):
    s, rq, sq, w = make(page_size=page_size, overlap=overlap)
    for i in range(12):
        rq.put(req(f"r{i}", 20 + 7 * i, n_out=5 + i))
    done = run(s, sq, 12)
    assert len(done) == 12
    for i in range(12):
        ids, fr = done[f"r{i}"]
        assert len(ids) == 5 + i and fr["type"] == "length"
    s.check_memory()       # raises on a leak
    assert s.req_to_token_pool.available_size() == s.req_to_token_pool.size


def test_outputs_independent_of_overlap_and_batching():
    outs = []
    for overlap, max_running in ((False, 64), (True, 64), (False, 2)):
        s, rq, sq, _ = make(page_size=16, overlap=overlap, max_running=max_running)
        for i in range(6):
            rq.put(req(f"r{i}", 30 + i, n_out=6, seed=i))
        done = run(s, sq, 6)
        outs.append({k: v[0] for k, v in done.items()})
    assert outs[0] == outs[1] == outs[2]


def test_chunked_prefill_splits_long_prompt():
    s, rq, sq, w = make(page_size=16, chunk=64)
    rq.put(req("long", 300, n_out=4))
    done = run(s, sq, 1)
    assert len(done["long"][0]) == 4
    ext = [b for b in w.batches if b.forward_mode.is_extend()]
    assert len(ext) == 5 and all(len(b.input_ids) <= 64 for b in ext)
    assert sum(len(b.input_ids) for b in ext) == 300
    s.check_memory()


def test_prefix_cache_hit_reduces_prefill():
    s, rq, sq, w = make(page_size=16)
    shared = list(range(100, 164))
    rq.put(req("a", 0, n_out=2, ids=shared + [1, 2, 3]))
    run(s, sq, 1)
    n_before = len(w.batches)
    rq.put(req("b", 0, n_out=2, ids=shared + [4, 5, 6, 7]))
    run(s, sq, 1)
    ext = [b for b in w.batches[n_before:] if b.forward_mode.is_extend()][0]
    assert int(ext.extend_prefix_lens[0]) == 64 and len(ext.input_ids) == 4
    s.check_memory()


def test_retract_on_memory_pressure_completes_all():
    # the admission estimate (new_token_ratio < 1) over-commits the pool on purpose
    s, rq, sq, w = make(page_size=1, max_total=300, max_running=8)
    for i in range(6):
        rq.put(req(f"r{i}", 10, n_out=100, seed=i))
    done = run(s, sq, 6, max_steps=20000)
    assert len(done) == 6 and all(len(v[0]) == 100 for v in done.values())
    assert s.total_retracted_reqs > 0
    s.check_memory()


def test_forced_retract_fault_injection(monkeypatch):
    import sglang_jax_b200.managers.scheduler as sch
    monkeypatch.setattr(sch, "TEST_RETRACT", True)
    monkeypatch.setattr(sch, "TEST_RETRACT_INTERVAL", 3)
    ref_s, rq, sq, _ = make(page_size=16)
    for i in range(4):
        rq.put(req(f"r{i}", 33, n_out=12, seed=i))
    got = run(ref_s, sq, 4, max_steps=20000)
    assert ref_s.total_retracted_reqs > 0
    monkeypatch.setattr(sch, "TEST_RETRACT", False)
    s2, rq2, sq2, _ = make(page_size=16)
    for i in range(4):
        rq2.put(req(f"r{i}", 33, n_out=12, seed=i))
    want = run(s2, sq2, 4)
    # retraction re-prefills over prompt + output: results are identical, the server survives
    assert {k: v[0] for k, v in got.items()} == {k: v[0] for k, v in want.items()}
    ref_s.check_memory()


@pytest.mark.parametrize("overlap", [False, True])
def test_abort_waiting_running_and_all(overlap):
    s, rq, sq, _ = make(page_size=16, overlap=overlap, max_running=2)
    for i in range(4):
        rq.put(req(f"r{i}", 40, n_out=200, seed=i))
    step = s.step_overlap if overlap else s.step_normal
    for _ in range(6):
        step()
    rq.put(AbortReq(rid="r3"))        # still waiting (max_running=2)
    rq.put(AbortReq(rid="r0"))        # running
    done = run(s, sq, 2, max_steps=50)
    assert done["r3"][1]["type"] == "abort" and done["r0"][1]["type"] == "abort"
    rq.put(AbortReq(abort_all=True))
    done2 = run(s, sq, 2, max_steps=50)
    assert all(v[1]["type"] == "abort" for v in done2.values())
    for _ in range(5):
        step()
    s.check_memory()


def test_abort_during_chunked_prefill():
    s, rq, sq, _ = make(page_size=16, chunk=64)
    rq.put(req("long", 500, n_out=4))
    s.step_normal()
    s.step_normal()
    assert s.chunked_req is not None
    rq.put(AbortReq(rid="long"))
    done = run(s, sq, 1, max_steps=20)
    assert done["long"][1]["type"] == "abort"
    s.check_memory()


@pytest.mark.parametrize("mode", ["abort", "retract", "in_place"])
def test_pause_continue(mode):
    s, rq, sq, _ = make(page_size=16)
    for i in range(3):
        rq.put(req(f"r{i}", 30, n_out=40, seed=i))
    for _ in range(5):
        s.step_normal()
    rq.put(PauseGenerationReqInput(mode=mode))
    ct = None
    for _ in range(5):
        s.step_normal()
        ct = ct if ct is not None else s.forward_ct
    assert s.forward_ct == ct          # no forward while paused
    rq.put(ContinueGenerationReqInput())
    done = run(s, sq, 3, max_steps=2000)
    if mode == "abort":
        assert all(v[1]["type"] == "abort" for v in done.values())
    else:
        assert all(v[1]["type"] == "length" and len(v[0]) == 40 for v in done.values())
    s.check_memory()


def test_flush_cache_only_when_idle():
    s, rq, sq, _ = make(page_size=16)
    rq.put(req("a", 64, n_out=50))
    for _ in range(3):
        s.step_normal()
    ok, _ = s.flush_cache()
    assert not ok
    run(s, sq, 1)
    assert s.tree_cache.total_size() > 0
    ok, n = s.flush_cache()
    assert ok and n > 0 and s.tree_cache.total_size() == 0
    assert s.token_to_kv_pool_allocator.available_size() == s.max_total_num_tokens // 16 * 16


def test_input_too_long_is_rejected():
    s, rq, sq, _ = make(ctx=128)
    rq.put(req("big", 500, n_out=4))
    done = run(s, sq, 1, max_steps=10)
    assert done["big"][1]["type"] == "abort" and done["big"][1]["status_code"] == 400


def test_stop_token_and_stream_interval():
    s, rq, sq, w = make()
    r = req("s", 10, n_out=30, seed=1)
    r.stream = True
    rq.put(r)
    chunks = []
    for _ in range(60):
        s.step_normal()
        while not sq.empty():
            o = sq.get()
            chunks.append((len(o.output_ids[0]), o.finished_reasons[0]))
    assert chunks[0][0] == 1 and chunks[-1][1] is not None and len(chunks) == 30
    # stop on a token id
    first_tok = None
    s2, rq2, sq2, _ = make()
    r2 = req("t", 10, n_out=30, seed=1)
    r2.sampling_params.ignore_eos = False
    r2.sampling_params.stop_token_ids = {chunks and 0}
    rq2.put(r2)
    done = run(s2, sq2, 1)
    assert done["t"][1]["type"] in ("stop", "length")
