"""End-to-end plumbing on CPU in fp32: the tiny Qwen3 config (2 layers, hidden 256, 4q/2kv heads,
head_dim 64 + q/k norm, FFN 512, vocab 1024, tied embeddings, page 16, radix cache on, 8 requests of
which 4 share a 64-token prefix, greedy, 32 new tokens) must reproduce HF transformers' Qwen3 tokens
exactly, independent of radix cache, chunking, overlap scheduling and tensor parallelism."""

import os
import sys
import time

import numpy as np
import pytest
import torch

from sglang_jax_b200.utils.tiny_models import TINY_QWEN3, tiny_qwen3_state_dict, write_tiny_qwen3_checkpoint

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def workload():
    rng = np.random.RandomState(0)
    prefix = rng.randint(0, 1024, size=64).tolist()
    reqs = []
    for i in range(8):
        n = int(rng.randint(32, 129))
        ids = rng.randint(0, 1024, size=n).tolist()
        if i < 4:
            ids = prefix + ids[: max(n - 64, 8)]
        reqs.append(ids)
    return reqs


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    return write_tiny_qwen3_checkpoint(str(tmp_path_factory.mktemp("tiny_qwen3")))


@pytest.fixture(scope="module")
def oracle():
    from transformers import Qwen3Config, Qwen3ForCausalLM
    cfg = Qwen3Config(**{k: v for k, v in TINY_QWEN3.items() if k not in ("architectures", "torch_dtype")})
    m = Qwen3ForCausalLM(cfg).float().eval()
    sd = tiny_qwen3_state_dict()
    sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
    m.load_state_dict(sd, strict=False)
    outs = []
    for ids in workload():
        with torch.no_grad():
            outs.append(m.generate(torch.tensor([ids]), max_new_tokens=32, do_sample=False)[0, len(ids):].tolist())
    return outs


def run_engine(ckpt, **kw):
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    ps.reset_state()
    args = dict(model_path=ckpt, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                max_total_tokens=8192, enable_single_process=True, max_running_requests=16)
    args.update(kw)
    eng = Engine(**args)
    try:
        outs = eng.generate(input_ids=workload(), sampling_params={"max_new_tokens": 32, "temperature": 0.0,
                                                                    "ignore_eos": True})
        info = eng.get_server_info()["internal_states"][0]
        return [o["output_ids"] for o in outs], [o["meta_info"]["cached_tokens"] for o in outs], info
    finally:
        eng.shutdown()


def test_matches_hf_oracle_with_radix_cache(ckpt, oracle):
    outs, cached, _ = run_engine(ckpt)
    assert outs == oracle


@pytest.mark.parametrize("kw", [
    dict(disable_radix_cache=True),
    dict(disable_overlap_schedule=True),
    dict(chunked_prefill_size=48, page_size=16),
    dict(page_size=1),
    dict(enable_mixed_chunk=True, chunked_prefill_size=64),
    dict(max_running_requests=3),
    dict(schedule_policy="lpm"),
    dict(enable_unified_radix_tree=True),
    dict(enable_unified_radix_tree=True, hicache_storage="host"),
])
def test_outputs_invariant_to_scheduling_options(ckpt, oracle, kw):
    outs, _, _ = run_engine(ckpt, **kw)
    assert outs == oracle


@pytest.mark.parametrize("unified", [False, True])
def test_prefix_cache_hits_are_reported(ckpt, unified):
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    ps.reset_state()
    eng = Engine(model_path=ckpt, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                 max_total_tokens=8192, enable_single_process=True, enable_unified_radix_tree=unified)
    try:
        # --enable-unified-radix-tree: the unified tree (FULL component alone for this model) shares prefixes alike
        assert (type(eng.scheduler.tree_cache).__name__ == "UnifiedRadixCache") == unified
        reqs = workload()
        sp = {"max_new_tokens": 4, "temperature": 0.0, "ignore_eos": True}
        first = eng.generate(input_ids=reqs[0], sampling_params=sp)
        second = eng.generate(input_ids=reqs[1], sampling_params=sp)
        assert first["meta_info"]["cached_tokens"] == 0
        assert second["meta_info"]["cached_tokens"] == 64       # the shared prefix: 4 pages of 16
    finally:
        eng.shutdown()


def _tp_rank(rank, world, port, ckpt, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, ROOT)
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.server_args import ServerArgs
    torch.set_num_threads(2)
    ps.init_distributed(rank, world, "cpu", init_method=f"tcp://127.0.0.1:{port}", timeout_s=120)
    sa = ServerArgs(model_path=ckpt, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                    max_total_tokens=8192, enable_single_process=True, max_running_requests=16, tp_size=world,
                    log_level="error", watchdog_timeout=0)
    if rank != 0:
        from sglang_jax_b200.managers.tp_worker import run_tp_follower
        run_tp_follower(sa)
    else:
        from sglang_jax_b200 import Engine
        eng = Engine(server_args=sa)
        want = os.environ.get("SGLB_EXPECT_TRANSPORT")
        if want:
            assert eng.scheduler.tp_worker.channel.transport == want, eng.scheduler.tp_worker.channel.transport
        outs = eng.generate(input_ids=workload(), sampling_params={"max_new_tokens": 32, "temperature": 0.0,
                                                                    "ignore_eos": True})
        q.put([o["output_ids"] for o in outs])
        eng.shutdown()
    ps.destroy()


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_gloo_matches_oracle(ckpt, oracle, world):
    """world 4 exceeds the model's two KV heads: they are replicated across rank pairs."""
    import torch.multiprocessing as mp
    from sglang_jax_b200.utils.common import get_free_port
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = get_free_port()
    procs = [ctx.Process(target=_tp_rank, args=(r, world, port, ckpt, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        outs = q.get(timeout=300)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    assert outs == oracle


def test_tensor_parallel_over_the_pubsub_mirror(ckpt, oracle, monkeypatch):
    """The multi-node form of the step hand-over on one machine: rank 0 publishes every step on a ZMQ PUB socket, the
    other rank subscribes (probe hand-shake, sequence numbers); same tokens as the oracle."""
    import torch.multiprocessing as mp
    from sglang_jax_b200.utils.common import get_free_port
    monkeypatch.setenv("SGLB_STEP_CHANNEL", "zmq")
    monkeypatch.setenv("SGLB_EXPECT_TRANSPORT", "zmq-pubsub")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = get_free_port()
    procs = [ctx.Process(target=_tp_rank, args=(r, 2, port, ckpt, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        outs = q.get(timeout=300)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    assert outs == oracle


# ------------------------------------------------------------------------------------------
# rank 0 -> follower step channel (shared-memory ring) and what happens when a follower dies
def test_step_channel_codec_roundtrip():
    import numpy as np
    from sglang_jax_b200.managers.schedule_batch import ForwardMode, ModelWorkerBatch, ModelWorkerSamplingInfo
    from sglang_jax_b200.parallel.step_channel import decode_batch, encode_batch
    B, T = 3, 7
    si = ModelWorkerSamplingInfo(temperatures=np.array([0.0, 0.7, 1.0], np.float32), top_ps=np.array([1, 0.9, 0.5], np.float32),
                                 top_ks=np.array([1, 40, 1 << 30], np.int32), min_ps=np.zeros(3, np.float32),
                                 sampling_seeds=np.array([5, 6, 7], np.int32), is_all_greedy=False,
                                 need_top_p_sampling=True, need_top_k_sampling=True, need_min_p_sampling=False,
                                 positions=np.array([4, 9, 2], np.int32))
    b = ModelWorkerBatch(bid=11, forward_mode=ForwardMode.EXTEND, input_ids=np.arange(T, dtype=np.int32) - 3,
                         req_pool_indices=np.array([2, 0, 5], np.int32), seq_lens=np.array([9, 3, 4], np.int32),
                         out_cache_loc=np.arange(T, dtype=np.int32) + 64, positions=np.arange(T, dtype=np.int32),
                         extend_prefix_lens=np.array([6, 0, 2], np.int32), extend_seq_lens=np.array([3, 3, 1], np.int32),
                         page_delta_rows=np.array([2, 5], np.int32), page_delta_pos=np.array([0, 1], np.int32),
                         page_delta_ids=np.array([9, 8], np.int32), sampling_info=si,
                         future_slots=np.array([3, 1, 6], np.int64), real_bs=3)
    ints = encode_batch(b)
    assert ints is not None and ints.dtype == np.int32
    d = decode_batch(ints)
    for f in ("input_ids", "req_pool_indices", "seq_lens", "out_cache_loc", "positions", "extend_prefix_lens",
              "extend_seq_lens", "page_delta_rows", "page_delta_pos", "page_delta_ids", "future_slots"):
        assert np.array_equal(getattr(d, f), getattr(b, f)), f
    assert d.future_slots.dtype == np.int64 and d.bid == 11 and d.forward_mode == ForwardMode.EXTEND
    for f in ("temperatures", "top_ps", "top_ks", "min_ps", "sampling_seeds", "positions"):
        assert np.array_equal(getattr(d.sampling_info, f), getattr(si, f)), f
    assert d.sampling_info.need_top_p_sampling and not d.sampling_info.is_all_greedy
    b.return_logprob = True          # anything beyond a plain step's integers travels pickled
    assert encode_batch(b) is None


def _ring_consumer(name, idx, n, q):
    sys.path.insert(0, ROOT)
    from sglang_jax_b200.mem_cache import _sched_native as sn
    ring = sn.StepRing(name, 4, 4096, 2, idx)
    got = []
    while len(got) < n:
        m = ring.pop(5.0, True)
        if m is None:
            break
        got.append((int(m[0]), bytes(m[1]) if m[0] == 0 else [int(x) for x in m[1]]))
    q.put((idx, got))


def test_step_ring_two_consumers_and_backpressure():
    import multiprocessing as mp
    import numpy as np
    from sglang_jax_b200.mem_cache import _sched_native as sn
    name = f"/sglb_test_ring_{os.getpid()}"
    ring = sn.StepRing(name, 4, 4096, 2)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    n = 20
    procs = [ctx.Process(target=_ring_consumer, args=(name, i, n, q)) for i in range(2)]
    for p in procs:
        p.start()
    for i in range(n):            # more messages than slots: the producer waits for both readers
        if i % 2:
            assert ring.push(b"msg%d" % i, 0, 10.0)
        else:
            assert ring.push_ints(np.arange(i, i + 3, dtype=np.int32), 1, 10.0)
    res = dict(q.get(timeout=30) for _ in range(2))
    for p in procs:
        p.join(timeout=10)
    want = [(0, b"msg%d" % i) if i % 2 else (1, [i, i + 1, i + 2]) for i in range(n)]
    assert res[0] == want and res[1] == want
    # nobody reads any more: the ring fills and a bounded push reports it instead of blocking
    for _ in range(4):
        assert ring.push(b"x", 0, 0.2)
    assert not ring.push(b"x", 0, 0.2)
    assert ring.slowest()[1] == 4


def _tp_rank_dies(rank, world, port, ckpt, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, ROOT)
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.server_args import ServerArgs
    torch.set_num_threads(2)
    ps.init_distributed(rank, world, "cpu", init_method=f"tcp://127.0.0.1:{port}", timeout_s=20)
    sa = ServerArgs(model_path=ckpt, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                    max_total_tokens=8192, enable_single_process=True, max_running_requests=16, tp_size=world,
                    log_level="critical", watchdog_timeout=0, dist_timeout=5)
    if rank != 0:
        from sglang_jax_b200.managers.tp_worker import run_tp_follower
        seen = {"n": 0}

        def die_mid_stream():
            seen["n"] += 1
            if seen["n"] >= 12:          # between two steps: nothing of this rank is in flight
                os._exit(0)

        run_tp_follower(sa, on_message=die_mid_stream)
        return
    from sglang_jax_b200 import Engine
    eng = Engine(server_args=sa)
    t0 = time.time()
    try:
        outs = eng.generate(input_ids=workload(), sampling_params={"max_new_tokens": 200, "temperature": 0.0,
                                                                    "ignore_eos": True})
        q.put(("finished", [len(o["output_ids"]) for o in outs], time.time() - t0))
    except Exception as e:
        q.put(("failed", f"{type(e).__name__}: {e}", time.time() - t0))
    q.close()
    q.join_thread()          # the result must leave this process before it exits without clean-up
    os._exit(0)


def test_follower_death_fails_pending_requests(ckpt):
    """A follower rank exits between two steps.  Rank 0 learns of it on the host (its next host collective
    errors out, or the step ring fills up) and fails the requests in flight instead of hanging."""
    import torch.multiprocessing as mp
    from sglang_jax_b200.utils.common import get_free_port
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = get_free_port()
    procs = [ctx.Process(target=_tp_rank_dies, args=(r, 2, port, ckpt, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        kind, detail, waited = q.get(timeout=240)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    assert kind == "failed", (kind, detail)
    assert waited < 200, waited


# ------------------------------------------------------------------------------------------
# penalties: token counts live with the model runner and are updated from each step's input ids
def _penalised_oracle(prompts, n_new, freq, pres, min_new, stop_id):
    from transformers import Qwen3Config, Qwen3ForCausalLM
    cfg = Qwen3Config(**{k: v for k, v in TINY_QWEN3.items() if k not in ("architectures", "torch_dtype")})
    m = Qwen3ForCausalLM(cfg).float().eval()
    sd = tiny_qwen3_state_dict()
    sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
    m.load_state_dict(sd, strict=False)
    outs = []
    for ids in prompts:
        cur, gen = list(ids), []
        counts = torch.zeros(1024)
        for _ in range(n_new):
            with torch.no_grad():
                lg = m(torch.tensor([cur])).logits[0, -1].float()
            lg = lg - freq * counts - pres * (counts > 0).float()
            if len(gen) < min_new:
                lg[stop_id] = float("-inf")
            t = int(lg.argmax())
            gen.append(t)
            cur.append(t)
            counts[t] += 1
            if t == stop_id:
                break
        outs.append(gen)
    return outs


@pytest.mark.parametrize("overlap", [False, True])
def test_frequency_presence_penalties_and_min_new_tokens_match_a_manual_oracle(ckpt, overlap):
    """Greedy decoding with penalties against HF logits penalised by hand: fresh requests, a batch that mixes
    penalised and plain requests, both schedules (with overlap the host does not know the last token when it
    builds the next step: the counts are updated on the device from the step's own input ids)."""
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    prompts = workload()[:4]
    freq, pres, n_new = 0.9, 0.6, 24
    plain = _penalised_oracle(prompts, n_new, 0.0, 0.0, 0, -1)
    want = _penalised_oracle(prompts, n_new, freq, pres, 0, -1)
    assert want != plain                                           # the penalties change these sequences
    stop = plain[0][2]                                             # a token the plain run emits early
    want_min = _penalised_oracle(prompts[:1], n_new, 0.0, 0.0, 6, stop)[0]
    assert stop not in want_min[:6]
    ps.reset_state()
    eng = Engine(model_path=ckpt, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                 max_total_tokens=8192, enable_single_process=True, max_running_requests=16,
                 disable_overlap_schedule=not overlap, log_level="error")
    try:
        sp = {"max_new_tokens": n_new, "temperature": 0.0, "ignore_eos": True}
        pen = dict(sp, frequency_penalty=freq, presence_penalty=pres)
        got = eng.generate(input_ids=prompts, sampling_params=[pen, pen, sp, pen])
        assert [o["output_ids"] for o in got] == [want[0], want[1], plain[2], want[3]]
        # min_new_tokens: the stop token is suppressed for the first six tokens, then ends the request
        r = eng.generate(input_ids=prompts[0], sampling_params={"max_new_tokens": n_new, "temperature": 0.0,
                                                                "min_new_tokens": 6, "stop_token_ids": [stop]})
        assert r["output_ids"] == want_min and len(want_min) >= 6
        # the slot's counts are reset when another request reuses it
        again = eng.generate(input_ids=prompts[:2], sampling_params=pen)
        assert [o["output_ids"] for o in again] == want[:2]
    finally:
        eng.shutdown()


def test_several_engines_in_one_process_keep_their_own_parallel_state(ckpt, oracle):
    """`device_indexes` pins a single-process engine to one device; its scheduler thread carries its own parallel
    state, so two engines of one process (RL roll-out workers) do not disturb each other or the process-wide state
    (reference `test/srt/rl/test_multi_engines_in_one_process.py`)."""
    import threading
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    ps.reset_state()
    kw = dict(model_path=ckpt, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
              max_total_tokens=8192, enable_single_process=True)
    a = Engine(device_indexes=[0], **kw)
    b = Engine(device_indexes=[1], **kw)
    try:
        assert a.parallel_state is not b.parallel_state and not ps.get_state().initialized
        assert a.parallel_state.local_rank == 0 and a.parallel_state.initialized
        sp = {"max_new_tokens": 32, "temperature": 0.0, "ignore_eos": True}
        res = {}
        ts = [threading.Thread(target=lambda n=n, e=e: res.update({n: e.generate(input_ids=workload(), sampling_params=sp)}))
              for n, e in (("a", a), ("b", b))]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=300)
        assert [o["output_ids"] for o in res["a"]] == oracle and [o["output_ids"] for o in res["b"]] == oracle
        assert res["a"][0]["meta_info"].get("cache_miss_count", 0) == 0
    finally:
        a.shutdown()
        b.shutdown()


def test_tokenizer_batch_encode_tokenizes_a_batch_in_one_call(ckpt):
    """`--enable-tokenizer-batch-encode`: the texts of a batch request go through the tokenizer in one call and
    produce the outputs of the per-request path; token-id inputs are refused under the flag."""
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps

    class Tok:
        eos_token_id = None
        calls = []

        def encode(self, text, **kw):
            self.calls.append(("one", text))
            return [5 + (ord(c) % 200) for c in text]

        def __call__(self, texts, **kw):
            self.calls.append(("batch", len(texts)))
            return {"input_ids": [[5 + (ord(c) % 200) for c in t] for t in texts]}

        def decode(self, ids, **kw):
            return " ".join(map(str, ids))

    ps.reset_state()
    eng = Engine(model_path=ckpt, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                 max_total_tokens=8192, enable_single_process=True)
    try:
        tok = Tok()
        eng.tokenizer_manager.tokenizer = tok
        texts = ["the quick brown fox", "jumps over", "the lazy dog again and again"]
        sp = {"max_new_tokens": 6, "temperature": 0.0, "ignore_eos": True}
        want = [o["output_ids"] for o in eng.generate(prompt=texts, sampling_params=sp)]
        assert [c[0] for c in tok.calls] == ["one"] * 3
        tok.calls.clear()
        eng.tokenizer_manager.server_args.enable_tokenizer_batch_encode = True
        got = [o["output_ids"] for o in eng.generate(prompt=texts, sampling_params=sp)]
        assert got == want and tok.calls == [("batch", 3)]
        with pytest.raises(Exception, match="pre-tokenized"):
            eng.generate(input_ids=[[5, 6, 7], [8, 9]], sampling_params=sp)
    finally:
        eng.shutdown()


def test_engine_loop_daemon_lets_threads_generate_concurrently(ckpt, oracle):
    """`--enable-engine-loop-run-forever-daemon`: the engine's event loop turns on its own thread and the synchronous
    `generate` only hands it coroutines, so several threads can call it at once (without the flag the loop belongs to
    the calling thread and a second concurrent call is an error)."""
    import threading
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    ps.reset_state()
    eng = Engine(model_path=ckpt, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                 max_total_tokens=8192, enable_single_process=True, enable_engine_loop_run_forever_daemon=True)
    try:
        reqs = workload()
        sp = {"max_new_tokens": 32, "temperature": 0.0, "ignore_eos": True}
        res = [None] * len(reqs)

        def one(i):
            res[i] = eng.generate(input_ids=reqs[i], sampling_params=sp)["output_ids"]

        ts = [threading.Thread(target=one, args=(i,)) for i in range(len(reqs))]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=300)
        assert res == oracle
        assert [c["output_ids"] for c in eng.generate(input_ids=reqs[0], sampling_params=sp, stream=True)][-1] == oracle[0]
        assert eng.get_server_info()["internal_states"]
    finally:
        eng.shutdown()
    assert eng._loop_thread is None


def test_dtype_config_sets_per_module_parameter_dtypes(ckpt, oracle, tmp_path):
    """`--dtype-config`: a nested mapping of module names to dtypes; missing keys fall back to the level's default,
    fused projections follow their first member, and a layer with a different weight dtype computes in it."""
    import json
    import torch
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.configs.dtype_config import DtypeConfig
    from sglang_jax_b200.parallel import state as ps
    cfg = {"model": {"norm": "bfloat16", "layers": {"input_layernorm": "bfloat16",
                                                     "self_attn": {"q_proj": "bfloat16"},
                                                     "mlp": {"down_proj": "bfloat16"}}}}
    d = DtypeConfig(cfg, default_dtype="float32")
    assert d.resolve("model.layers.3.self_attn.qkv_proj.weight") == torch.bfloat16           # via q_proj
    assert d.resolve("model.layers.0.self_attn.o_proj.weight") == torch.float32
    assert d.resolve("model.layers.1.mlp.gate_up_proj.weight") == torch.float32
    assert d.resolve("lm_head.weight") == torch.float32 and d.resolve("model.norm.weight") == torch.bfloat16
    assert d.get_config("model").get_config("layers").get_optional_dtype("softmax") is None
    with pytest.raises(ValueError):
        DtypeConfig({"model": "float7"})
    path = tmp_path / "dt.json"
    path.write_text(json.dumps(cfg))
    ps.reset_state()
    eng = Engine(model_path=ckpt, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                 max_total_tokens=8192, enable_single_process=True, dtype_config=str(path))
    try:
        params = dict(eng.scheduler.tp_worker.model_runner.model.named_parameters())
        assert params["model.layers.0.self_attn.qkv_proj.weight"].dtype == torch.bfloat16
        assert params["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
        assert params["model.layers.0.input_layernorm.weight"].dtype == torch.bfloat16
        assert params["model.layers.0.self_attn.o_proj.weight"].dtype == torch.float32
        assert params["model.layers.0.post_attention_layernorm.weight"].dtype == torch.float32
        outs = eng.generate(input_ids=workload(), sampling_params={"max_new_tokens": 8, "temperature": 0.0,
                                                                   "ignore_eos": True})
        got = [o["output_ids"] for o in outs]
        # bf16 weights in a few layers: same length, first tokens mostly those of the all-fp32 model
        assert all(len(g) == 8 for g in got)
        assert sum(g[:2] == w[:2] for g, w in zip(got, oracle)) >= len(oracle) // 2
    finally:
        eng.shutdown()
