"""Data-parallel attention under one scheduler: routing, per-section pools and trees, lock-step loop, and the
multi-process form where other sections' leaders are fed through shared-memory rings."""

import queue

import numpy as np
import pytest

from sglang_jax_b200.managers.dp_scheduler import DPScheduler
from sglang_jax_b200.managers.io_struct import AbortReq, FlushCacheReqInput, TokenizedGenerateReqInput
from sglang_jax_b200.managers.scheduler import Scheduler
from sglang_jax_b200.managers.tp_worker import MockModelWorker
from sglang_jax_b200.sampling.sampling_params import SamplingParams
from sglang_jax_b200.server_args import ServerArgs


def _args(dp, overlap, policy="round_robin", **kw):
    return ServerArgs(model_path="mock", device="cpu", page_size=4, skip_tokenizer_init=True, dp_size=dp, tp_size=dp,
                      disable_overlap_schedule=not overlap, dp_schedule_policy=policy, max_running_requests=16, **kw)


def _worker(sa, total=512):
    return MockModelWorker(sa, max_total_num_tokens=total, max_running_requests=16, context_len=256, page_size=4)


def _req(rid, ids, n_out=6, **kw):
    return TokenizedGenerateReqInput(rid=rid, input_ids=list(ids), sampling_params=SamplingParams(
        max_new_tokens=n_out, temperature=0.0, ignore_eos=True), **kw)


def _drain(step, sq, n, max_steps=4000):
    done, ranks = {}, {}
    for _ in range(max_steps):
        step()
        while not sq.empty():
            o = sq.get()
            if not hasattr(o, "rids"):
                done.setdefault("_ctl", []).append(o)
                continue
            for i, (rid, ids, fr) in enumerate(zip(o.rids, o.output_ids, o.finished_reasons)):
                if fr is not None:
                    done[rid] = ids
                    if o.dp_ranks:
                        ranks[rid] = o.dp_ranks[i]
        if len([k for k in done if k != "_ctl"]) >= n:
            break
    for _ in range(4):
        step()
    return done, ranks


@pytest.mark.parametrize("overlap", [False, True])
def test_sections_match_single_scheduler_and_keep_their_own_pools(overlap):
    rng = np.random.RandomState(0)
    prompts = [rng.randint(1, 900, size=n).tolist() for n in (12, 30, 7, 19, 25, 9, 40, 5)]
    sa1 = _args(1, overlap)
    rq, sq = queue.Queue(), queue.Queue()
    one = Scheduler(sa1, None, tp_worker=_worker(sa1), recv_queue=rq, send_queue=sq)
    for i, p in enumerate(prompts):
        rq.put(_req(f"r{i}", p))
    want, _ = _drain(one.step_overlap if overlap else one.step_normal, sq, len(prompts))

    sa = _args(2, overlap)
    workers = [_worker(sa), _worker(sa)]
    rq, sq = queue.Queue(), queue.Queue()
    dp = DPScheduler(sa, None, workers, recv_queue=rq, send_queue=sq)
    assert dp.max_total_num_tokens == 1024 and len(dp.sections) == 2
    for i, p in enumerate(prompts):
        rq.put(_req(f"r{i}", p))
    got, ranks = _drain(dp.step, sq, len(prompts))
    assert {k: v for k, v in got.items() if k != "_ctl"} == {k: v for k, v in want.items() if k != "_ctl"}
    assert [ranks[f"r{i}"] for i in range(8)] == [0, 1] * 4 and dp.routed == [4, 4]
    # each section ran its own batches on its own worker, with its own allocator and tree
    assert workers[0].forward_ct > 0 and workers[1].forward_ct > 0
    a0, a1 = (s.token_to_kv_pool_allocator for s in dp.sections)
    assert a0 is not a1 and dp.sections[0].tree_cache is not dp.sections[1].tree_cache
    for s in dp.sections:
        s.check_memory()
        assert s.token_to_kv_pool_allocator.available_size() + s.tree_cache.evictable_size() == s.max_total_num_tokens


def test_pinned_rank_cache_aware_routing_abort_and_flush():
    sa = _args(2, False, policy="cache_aware")
    rq, sq = queue.Queue(), queue.Queue()
    dp = DPScheduler(sa, None, [_worker(sa), _worker(sa)], recv_queue=rq, send_queue=sq)
    shared = list(range(100, 164))
    rq.put(_req("warm", shared + [1, 2, 3], dp_rank=1))
    got, ranks = _drain(dp.step, sq, 1)
    assert ranks["warm"] == 1
    # the prefix now sits in section 1's tree only: cache-aware routing follows it, other prompts go to the
    # lighter section
    rq.put(_req("hit", shared + [7, 8, 9, 10]))
    rq.put(_req("cold", list(range(500, 540))))
    got, ranks = _drain(dp.step, sq, 2)
    assert ranks["hit"] == 1 and ranks["cold"] == 0
    assert dp.sections[1].stats["num_cached_tokens"] >= 60 and dp.sections[0].stats["num_cached_tokens"] == 0
    # abort reaches whichever section holds the request
    rq.put(_req("long", list(range(300, 330)), n_out=200, dp_rank=1))
    for _ in range(5):
        dp.step()
    rq.put(AbortReq(rid="long"))
    got, ranks = _drain(dp.step, sq, 1)
    assert "long" in got and len(got["long"]) < 200
    # flush empties every section's tree
    rq.put(FlushCacheReqInput())
    for _ in range(3):
        dp.step()
    assert all(s.tree_cache.evictable_size() == 0 for s in dp.sections)
    ctl = []
    while not sq.empty():
        ctl.append(sq.get())
    assert any(getattr(c, "success", False) for c in ctl)


@pytest.mark.parametrize("policy", ["min_running_queue", "shape_aware"])
def test_load_policies_balance_sections(policy):
    sa = _args(4, True, policy=policy)
    rq, sq = queue.Queue(), queue.Queue()
    dp = DPScheduler(sa, None, [_worker(sa) for _ in range(4)], recv_queue=rq, send_queue=sq)
    rng = np.random.RandomState(1)
    for i in range(24):
        rq.put(_req(f"r{i}", rng.randint(1, 900, size=int(rng.randint(4, 60))).tolist(), n_out=12))
        dp.step()
    got, ranks = _drain(dp.step, sq, 24)
    assert len(ranks) == 24 and max(dp.routed) - min(dp.routed) <= 4 and min(dp.routed) >= 3


def _mp_engine(tmp_path, dp, tp, prompts, sp, **kw):
    from sglang_jax_b200.entrypoints.engine import Engine
    eng = Engine(model_path=str(tmp_path / "m"), device="cpu", page_size=4, skip_tokenizer_init=True,
                 max_total_tokens=2048, dtype="float32", log_level="error", dp_size=dp, tp_size=tp,
                 dp_schedule_policy="round_robin", watchdog_timeout=0, **kw)
    try:
        outs = eng.generate(input_ids=prompts, sampling_params=sp)
        extra = eng.generate(input_ids=prompts[:2], sampling_params=sp, dp_rank=dp - 1, return_logprob=True,
                             top_logprobs_num=2)
        return outs, extra
    finally:
        eng.shutdown()


@pytest.mark.parametrize("world", [2, 4])
def test_processes_two_sections_match_single_engine(tmp_path, world):
    """dp 2 x tensor 1 (and dp 2 x tensor 2) as processes (gloo): the outputs of both sections equal a single engine's, requests
    alternate between the sections, a pinned `dp_rank` is honoured and log-probabilities travel back from the
    other section's leader."""
    from sglang_jax_b200.utils.tiny_models import write_tiny_qwen3_checkpoint
    write_tiny_qwen3_checkpoint(str(tmp_path / "m"))
    rng = np.random.RandomState(0)
    prompts = [rng.randint(5, 1000, size=n).tolist() for n in (12, 30, 7, 19, 25, 9)]
    sp = {"temperature": 0.0, "max_new_tokens": 6, "ignore_eos": True}
    want, want_lp = _mp_engine(tmp_path, 1, 1, prompts, sp)
    outs, lp = _mp_engine(tmp_path, 2, world, prompts, sp)
    assert [o["output_ids"] for o in outs] == [o["output_ids"] for o in want]
    assert [o["meta_info"]["dp_rank"] for o in outs] == [0, 1, 0, 1, 0, 1]
    assert [o["meta_info"]["dp_rank"] for o in lp] == [1, 1]
    for a, b in zip(lp, want_lp):
        assert a["output_ids"] == b["output_ids"]
        va = [x[0] for x in a["meta_info"]["output_token_logprobs"]]
        vb = [x[0] for x in b["meta_info"]["output_token_logprobs"]]
        np.testing.assert_allclose(va, vb, atol=1e-3)
        assert len(a["meta_info"]["output_top_logprobs"][0]) == 2
