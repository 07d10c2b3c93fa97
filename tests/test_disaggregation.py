"""PD disaggregation on CPU: control plane units (state machine, registry + heartbeats, auth,
reaper, watchdog, router) and an end-to-end prefill -> transfer -> decode run whose output
must equal a single engine's (reference tests: `python/sgl_jax/test/disaggregation/`).
Failures are injected on the host only: a peer that never answers, a dropped acknowledgement,
a wrong secret."""

import threading
import time

import numpy as np
import pytest
import torch

from sglang_jax_b200.disaggregation import pd_auth
from sglang_jax_b200.disaggregation.base.kv_manager import KVPoll, StateHolder
from sglang_jax_b200.disaggregation.bootstrap import (BootstrapClient, BootstrapServer, HeartbeatDaemon,
                                                      IncompatiblePeer, PrefillInfoCache, Registry, check_compat)
from sglang_jax_b200.disaggregation.common import metrics
from sglang_jax_b200.disaggregation.common.core import CommonKVManager
from sglang_jax_b200.disaggregation.debug_utils import kv_digest
from sglang_jax_b200.disaggregation.decode_watchdog import EventLoopWatchdog
from sglang_jax_b200.disaggregation.transfer.zmq_transfer import TransferError, ZmqTransferBackend
from sglang_jax_b200.mem_cache.memory_pool import MHATokenToKVPool
from sglang_jax_b200.utils.common import get_free_port


def test_state_machine_rejects_illegal_moves():
    s = StateHolder()
    with pytest.raises(ValueError):
        s.transition(KVPoll.TRANSFERRING)
    s.transition(KVPoll.WAITING_FOR_INPUT)
    s.transition(KVPoll.TRANSFERRING)
    s.transition(KVPoll.SUCCESS)
    with pytest.raises(ValueError):
        s.transition(KVPoll.FAILED)
    f = StateHolder()
    f.fail("peer vanished")
    assert f.state == KVPoll.FAILED and f.failure == "peer vanished"
    f.fail("again")      # terminal: ignored
    assert f.failure == "peer vanished"


def test_auth_tokens_and_tags():
    assert pd_auth.check_bearer(None, None)
    hdr = pd_auth.auth_headers("s3cret")["Authorization"]
    assert pd_auth.check_bearer(hdr, "s3cret") and not pd_auth.check_bearer(hdr, "other")
    assert not pd_auth.check_bearer(None, "s3cret")
    tag = pd_auth.sign(b"payload", "k")
    assert pd_auth.verify(b"payload", tag, "k") and not pd_auth.verify(b"payload!", tag, "k")


LAYOUT = {"page_size": 16, "num_layers": 2, "page_bytes_per_layer": [4096, 4096], "dtype": "float32", "tp_size": 1,
          "model": "Qwen3ForCausalLM"}


def test_registry_ttl_compat_and_protocol_floor():
    reg = Registry(ttl=0.15)
    reg.register(dict(LAYOUT, engine_id="p0", transfer_addr="h:1", protocol_version=3))
    with pytest.raises(IncompatiblePeer):
        reg.register(dict(LAYOUT, page_size=32, engine_id="p1", transfer_addr="h:2", protocol_version=3))
    with pytest.raises(IncompatiblePeer):
        reg.register(dict(LAYOUT, engine_id="p2", transfer_addr="h:3", protocol_version=1))
    assert len(reg.table()["prefills"]) == 1
    time.sleep(0.2)
    assert reg.table()["prefills"] == []                     # missed its heartbeats
    assert not reg.heartbeat("p0")
    with pytest.raises(IncompatiblePeer):
        check_compat(LAYOUT, dict(LAYOUT, dtype="bfloat16", protocol_version=3))


def test_bootstrap_http_heartbeat_and_cache():
    srv = BootstrapServer(port=get_free_port(), ttl=0.6, secret="abc").start()
    try:
        bad = BootstrapClient(srv.url, secret="wrong")
        with pytest.raises(Exception):
            bad.prefills()
        cl = BootstrapClient(srv.url, secret="abc")
        hb = HeartbeatDaemon(cl, dict(LAYOUT, engine_id="p0", tp_rank=0, transfer_addr="127.0.0.1:5", ack_addr="a:1",
                                      http_url="http://x"), interval=0.1).start()
        cache = PrefillInfoCache(cl, LAYOUT, refresh_interval=0.05)
        assert cache.lookup("p0")["transfer_addr"] == "127.0.0.1:5"
        assert cache.lookup(None, room=77)["engine_id"] == "p0"
        time.sleep(0.9)                                       # several TTLs: heartbeats keep it alive
        assert cache.lookup("p0") is not None and hb.beats >= 3
        srv.registry.unregister("p0")                         # registry forgot us (e.g. it restarted)
        time.sleep(0.3)
        assert hb.reregistrations >= 1 and cache.lookup("p0") is not None
        hb.stop()
        time.sleep(0.1)                                       # let the cached table age out
        assert cache.lookup("p0") is None
        other = PrefillInfoCache(cl, dict(LAYOUT, page_size=64), refresh_interval=0)
        assert other.engines() == []
    finally:
        srv.stop()


def _pool(seed=None):
    pool = MHATokenToKVPool(16 * 16, 16, torch.float32, 2, 8, 2, "cpu")
    if seed is not None:
        g = torch.Generator().manual_seed(seed)
        for b in pool.kv_buffer:
            b.copy_(torch.randn(b.shape, generator=g))
    return pool


def test_transfer_pull_ack_and_digest():
    metrics.reset()
    src, dst = _pool(1), _pool()
    page_bytes = sum(b[0].numel() * 4 for b in src.kv_buffer)
    pb = ZmqTransferBackend(src, secret="k")
    pb.start()
    pm = CommonKVManager("prefill", pb, page_bytes, secret="k", reaper_interval=0.05, ack_timeout=5)
    dm = CommonKVManager("decode", ZmqTransferBackend(dst, secret="k", pull_timeout=5), page_bytes, secret="k",
                         reaper_interval=0.05, pull_timeout=5)
    try:
        recv = dm.create_receiver("r1")
        recv.init(np.array([9, 3, 4]), "room-1", pb.addr)      # decode may ask before prefill is ready
        time.sleep(0.05)
        assert recv.poll() in (KVPoll.WAITING_FOR_INPUT, KVPoll.TRANSFERRING)
        send = pm.create_sender("r1")
        send.init(np.array([2, 5, 7]), "room-1", first_token=42, meta={"kv_len": 40})
        send.send()
        t0 = time.time()
        while time.time() - t0 < 5 and not (recv.poll().terminal and send.poll().terminal):
            time.sleep(0.01)
        assert recv.poll() == KVPoll.SUCCESS and send.poll() == KVPoll.SUCCESS
        assert recv.meta["first_token"] == 42 and recv.meta["kv_len"] == 40
        assert kv_digest(src, [2, 5, 7]) == kv_digest(dst, [9, 3, 4])
        assert "room-1" not in pb.registered                   # released after the acknowledgement
        snap = metrics.snapshot()
        assert any(k.startswith("pd_transfer_total") and "success" in k for k in snap)
        send.clear(), recv.clear()
        assert pm.drain(1) and dm.drain(1)
        with pytest.raises(RuntimeError):
            pm.create_sender("late")
    finally:
        pm.shutdown(), dm.shutdown()


def test_reaper_fails_orphans_and_wrong_secret_is_refused():
    src, dst = _pool(2), _pool()
    pb = ZmqTransferBackend(src, secret="k")
    pb.start()
    pm = CommonKVManager("prefill", pb, 1, secret="k", reaper_interval=0.05, ack_timeout=0.2)
    dm = CommonKVManager("decode", ZmqTransferBackend(dst, secret="nope", pull_timeout=0.5), 1, secret="nope",
                         reaper_interval=0.05, pull_timeout=0.5)
    try:
        # nobody ever pulls: the sender is reaped after ack_timeout and its pages are released
        s = pm.create_sender("orphan")
        s.init(np.array([1]), "room-x", 1)
        s.send()
        t0 = time.time()
        while time.time() - t0 < 3 and s.poll() != KVPoll.FAILED:
            time.sleep(0.02)
        assert s.poll() == KVPoll.FAILED and "acknowledgement" in s.state.failure and "room-x" not in pb.registered
        # a decode engine with the wrong secret cannot read pages
        s2 = pm.create_sender("guarded")
        s2.init(np.array([1]), "room-y", 1)
        s2.send()
        r = dm.create_receiver("guarded")
        r.init(np.array([3]), "room-y", pb.addr)
        t0 = time.time()
        while time.time() - t0 < 3 and not r.poll().terminal:
            time.sleep(0.02)
        assert r.poll() == KVPoll.FAILED and "unauthorized" in r.state.failure
        assert torch.count_nonzero(dst.kv_buffer[0][3]) == 0
        # a peer that is not there at all: bounded wait, then FAILED
        r2 = dm.create_receiver("nobody")
        r2.init(np.array([4]), "room-z", f"127.0.0.1:{get_free_port()}")
        t0 = time.time()
        while time.time() - t0 < 4 and not r2.poll().terminal:
            time.sleep(0.02)
        assert r2.poll() == KVPoll.FAILED and "timed out" in r2.state.failure
    finally:
        pm.shutdown(), dm.shutdown()


def test_decode_watchdog_flags_a_stalled_loop():
    stalls = []
    wd = EventLoopWatchdog(0.1, has_work=lambda: True, on_stall=stalls.append, poll=0.02).start()
    try:
        for _ in range(10):
            wd.beat()
            time.sleep(0.02)
        assert not stalls
        time.sleep(0.3)                 # the loop "hangs" (host-side stand-in: it simply stops beating)
        assert stalls and stalls[0] > 0.1
    finally:
        wd.stop()
    idle = EventLoopWatchdog(0.05, has_work=lambda: False, on_stall=stalls.append, poll=0.01).start()
    n = len(stalls)
    time.sleep(0.2)
    idle.stop()
    assert len(stalls) == n             # nothing pending: silence is fine


def test_router_policies_and_room_fanout():
    from sglang_jax_b200.disaggregation.mini_lb import MiniLoadBalancer, PrefillEndpoint
    from sglang_jax_b200.disaggregation.router_args import RouterArgs
    lb = MiniLoadBalancer(RouterArgs(prefill_urls=["http://p0", "http://p1"], decode_urls=["http://d0", "http://d1", "http://d2"]))
    picks = [lb.pick() for _ in range(6)]
    assert [p.http_url for p, _ in picks] == ["http://p0", "http://p1"] * 3
    assert [d for _, d in picks] == ["http://d0", "http://d1", "http://d2"] * 2
    lb.args.policy = "shortest_queue"
    lb.prefills[0].inflight = 5
    lb.decode_inflight["http://d0"] = 2
    p, d = lb.pick()
    assert p.http_url == "http://p1" and d == "http://d1"
    ep = PrefillEndpoint("http://p0", "10.0.0.1:30001", "e0")
    pre, dec = lb._augment({"input_ids": [[1, 2], [3, 4]], "stream": True}, ep, 100)
    assert pre["bootstrap_room"] == [100, 101] and pre["stream"] is False
    assert dec["bootstrap_host"] == ["10.0.0.1"] * 2 and dec["bootstrap_port"] == [30001] * 2 and dec["stream"]
    pre, dec = lb._augment({"text": "hi"}, ep, 7)
    assert pre["bootstrap_room"] == 7 and dec["bootstrap_host"] == "10.0.0.1"
    empty = MiniLoadBalancer(RouterArgs(decode_urls=["http://d0"]))
    with pytest.raises(RuntimeError):
        empty.pick()
    # --prefill-bootstrap-host rewrites the host the decode engine is told to pull from
    lb.args.prefill_bootstrap_host = "pod-7.internal"
    _, dec = lb._augment({"text": "hi"}, ep, 8)
    assert dec["bootstrap_host"] == "pod-7.internal" and dec["bootstrap_port"] == 30001
    # --max-concurrent-requests: a gate of that many slots; command lines of the reference launcher parse
    import argparse
    import asyncio
    ap = argparse.ArgumentParser()
    RouterArgs.add_cli_args(ap)
    ns = ap.parse_args(["--decode", "http://d0", "--mini-lb", "--pd-disaggregation", "--request-timeout-secs", "30",
                        "--max-concurrent-requests", "2", "--prefill-bootstrap-host", "h"])
    ra = RouterArgs.from_cli_args(ns)
    assert ra.request_timeout == 30.0 and ra.max_concurrent_requests == 2 and ra.prefill_bootstrap_host == "h"
    gated = MiniLoadBalancer(ra)
    running, peak = 0, 0

    async def fake(path, body):
        nonlocal running, peak
        running += 1
        peak = max(peak, running)
        await asyncio.sleep(0.02)
        running -= 1
        return 200, {}

    gated._forward = fake

    async def burst():
        await asyncio.gather(*[gated.forward("/generate", {}) for _ in range(6)])

    asyncio.run(burst())
    assert peak == 2


def test_end_to_end_prefill_transfer_decode_matches_single_engine(tmp_path):
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import write_tiny_qwen3_checkpoint
    ckpt = write_tiny_qwen3_checkpoint(str(tmp_path / "m"))
    rng = np.random.RandomState(1)
    prompts = [rng.randint(5, 1000, size=n).tolist() for n in (40, 17, 70)]
    sp = {"temperature": 0.0, "max_new_tokens": 8, "ignore_eos": True}
    common = dict(model_path=ckpt, device="cpu", enable_single_process=True, page_size=16, skip_tokenizer_init=True,
                  max_total_tokens=2048, dtype="float32", log_level="error")
    ps.reset_state()
    plain = Engine(**common)
    try:
        want = [o["output_ids"] for o in plain.generate(input_ids=prompts, sampling_params=sp)]
        sp_pen = dict(sp, frequency_penalty=1.2, presence_penalty=0.4)
        want_pen = plain.generate(input_ids=prompts[0], sampling_params=sp_pen)["output_ids"]
    finally:
        plain.shutdown()
    srv = BootstrapServer(port=get_free_port(), secret="pd").start()
    pd_kw = dict(disaggregation_bootstrap_url=srv.url, disaggregation_shared_secret="pd",
                 disaggregation_transfer_port=0, disaggregation_side_channel_port=0)
    prefill = Engine(**common, disaggregation_mode="prefill", chunked_prefill_size=32,
                     enable_request_time_stats_logging=True, **pd_kw)
    decode = Engine(**common, disaggregation_mode="decode", enable_request_time_stats_logging=True, **pd_kw)
    stats_lines = []
    import logging as _logging

    class _Grab(_logging.Handler):
        def emit(self, record):
            if "PD time stats" in record.getMessage():
                stats_lines.append(record.getMessage())

    grab = _Grab()
    _logging.getLogger("sglang_jax_b200.disaggregation.req_time_stats").addHandler(grab)
    _logging.getLogger("sglang_jax_b200.disaggregation.req_time_stats").setLevel(_logging.INFO)
    try:
        res = {}

        def run(name, eng):
            res[name] = eng.generate(input_ids=prompts, sampling_params=sp, bootstrap_room=[11, 12, 13])

        ts = [threading.Thread(target=run, args=("decode", decode)), threading.Thread(target=run, args=("prefill", prefill))]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=120)
        assert "decode" in res and "prefill" in res
        # the decode engine keeps overlap scheduling: a transferred request's first step is fed its host-known token
        assert decode.scheduler.enable_overlap and prefill.scheduler.enable_overlap
        assert [o["output_ids"] for o in res["decode"]] == want
        assert [o["output_ids"] for o in res["prefill"]] == [w[:1] for w in want]
        # both engines are clean afterwards: the prefill released the pages once they were acknowledged
        t0 = time.time()
        while time.time() - t0 < 5 and prefill.scheduler.disagg_prefill_inflight:
            time.sleep(0.02)
        assert prefill.scheduler.disagg_sent == 3 and decode.scheduler.disagg_received == 3
        # --enable-request-time-stats-logging: one line per request and role with the stage durations
        roles = [("role=prefill" in l, "role=decode" in l) for l in stats_lines]
        assert sum(p for p, _ in roles) == 3 and sum(d for _, d in roles) == 3
        assert any("transfer_start->transfer_done" in l for l in stats_lines)
        assert any("transfer_done->first_decode_step" in l and "total_s" in l for l in stats_lines)
        time.sleep(0.1)
        prefill.scheduler.check_memory()
        decode.scheduler.check_memory()
        # penalties follow a transferred request: its token counts are rebuilt on the decode engine's device state
        pen = {}
        tp = [threading.Thread(target=lambda: pen.update(d=decode.generate(input_ids=prompts[0], sampling_params=sp_pen,
                                                                          bootstrap_room=21))),
              threading.Thread(target=lambda: pen.update(p=prefill.generate(input_ids=prompts[0], sampling_params=sp_pen,
                                                                           bootstrap_room=21)))]
        for t in tp:
            t.start()
        for t in tp:
            t.join(timeout=120)
        assert pen["d"]["output_ids"] == want_pen and want_pen != want[0]
        # a request whose prefill never happens fails cleanly on the decode side (bounded pull)
        decode.scheduler.disagg_kv_manager.backend.pull_timeout = 0.5
        lost = decode.generate(input_ids=prompts[:1], sampling_params=sp, bootstrap_room=[999])[0]
        fr = lost["meta_info"]["finish_reason"]
        assert fr["type"] == "abort" and fr["err_type"] == "KVTransferError" and lost["output_ids"] == []
        time.sleep(0.1)
        decode.scheduler.check_memory()
    finally:
        from sglang_jax_b200.disaggregation.runtime import shutdown_disaggregation
        shutdown_disaggregation(prefill.scheduler, 1)
        shutdown_disaggregation(decode.scheduler, 1)
        prefill.shutdown()
        decode.shutdown()
        srv.stop()
        _logging.getLogger("sglang_jax_b200.disaggregation.req_time_stats").removeHandler(grab)


def test_tensor_parallel_engines_hand_over_every_ranks_shard(tmp_path):
    """Prefill and decode engines with two tensor ranks each (gloo processes): rank r of the decode engine pulls the
    KV heads of its shard from rank r of the prefill engine; the decoded tokens equal a single engine's."""
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import write_tiny_qwen3_checkpoint
    ckpt = write_tiny_qwen3_checkpoint(str(tmp_path / "m"))
    rng = np.random.RandomState(2)
    prompts = [rng.randint(5, 1000, size=n).tolist() for n in (40, 17, 70, 33)]
    sp = {"temperature": 0.0, "max_new_tokens": 8, "ignore_eos": True}
    common = dict(model_path=ckpt, device="cpu", page_size=16, skip_tokenizer_init=True, max_total_tokens=2048,
                  dtype="float32", log_level="error", watchdog_timeout=0)
    ps.reset_state()
    plain = Engine(**common, enable_single_process=True)
    try:
        want = [o["output_ids"] for o in plain.generate(input_ids=prompts, sampling_params=sp)]
    finally:
        plain.shutdown()
    srv = BootstrapServer(port=get_free_port(), secret="pd").start()
    pd_kw = dict(disaggregation_bootstrap_url=srv.url, disaggregation_shared_secret="pd",
                 disaggregation_transfer_port=0, disaggregation_side_channel_port=0, tp_size=2)
    prefill = Engine(**common, disaggregation_mode="prefill", chunked_prefill_size=32, **pd_kw)
    decode = Engine(**common, disaggregation_mode="decode", **pd_kw)
    try:
        res = {}

        def run(name, eng):
            res[name] = eng.generate(input_ids=prompts, sampling_params=sp, bootstrap_room=[21, 22, 23, 24])

        ts = [threading.Thread(target=run, args=("decode", decode)), threading.Thread(target=run, args=("prefill", prefill))]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=180)
        assert "decode" in res and "prefill" in res
        assert [o["output_ids"] for o in res["decode"]] == want
        assert [o["output_ids"] for o in res["prefill"]] == [w[:1] for w in want]
    finally:
        prefill.shutdown()
        decode.shutdown()
        srv.stop()


@pytest.mark.gpu
def test_host_staged_transfer_uses_the_queue_pool_on_gpu():
    """Host-staged (tcp) hand-over between two pools on a GPU: pages travel through the pinned `QueueHostKVPool`
    slots (reserve -> page-copy kernel -> frames -> page-copy kernel -> release); several transfers share the slots."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")

    def pool(seed=None):
        p = MHATokenToKVPool(16 * 16, 16, torch.bfloat16, 2, 64, 3, "cuda")
        if seed is not None:
            g = torch.Generator(device="cuda").manual_seed(seed)
            for b in p.kv_buffer:
                b.copy_(torch.randn(b.shape, generator=g, device="cuda"))
        return p

    src, dst = pool(3), pool()
    pb = ZmqTransferBackend(src, secret="k", staging_pages=4)
    db = ZmqTransferBackend(dst, secret="k", pull_timeout=10, staging_pages=4)
    assert pb.staging is not None and db.staging is not None and pb.staging.num_pages == 4
    pb.start()
    try:
        for i, (sp, dp) in enumerate((([2, 5, 7], [9, 3, 4]), ([1, 6], [10, 11]), ([8, 12, 13, 14], [1, 2, 5, 6]))):
            pb.register(f"t{i}", np.asarray(sp), {"first_token": i})
            head = db.pull(pb.addr, f"t{i}", np.asarray(dp))
            assert head["first_token"] == i
            assert kv_digest(src, sp) == kv_digest(dst, dp)
        assert pb.staging.available_pages() == 4 and db.staging.available_pages() == 4     # every slot came back
        # a transfer larger than the pool falls back to a one-off buffer
        pb.register("big", np.arange(1, 7), {})
        db.pull(pb.addr, "big", np.arange(7, 13))
        assert kv_digest(src, list(range(1, 7))) == kv_digest(dst, list(range(7, 13)))
    finally:
        pb.stop()


def test_embedded_bootstrap_server_and_decode_watchdog_flags(tmp_path, monkeypatch):
    """`DISAGG_LAUNCH_BOOTSTRAP=1`: the engine hosts the registry on `--disaggregation-bootstrap-port` and needs no
    URL; `--disaggregation-decode-watchdog-seconds` arms the loop watchdog of the decode engine."""
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import write_tiny_qwen3_checkpoint
    from sglang_jax_b200.disaggregation.runtime import shutdown_disaggregation
    ckpt = write_tiny_qwen3_checkpoint(str(tmp_path / "m"))
    port = get_free_port()
    monkeypatch.setenv("DISAGG_LAUNCH_BOOTSTRAP", "1")
    ps.reset_state()
    common = dict(model_path=ckpt, device="cpu", enable_single_process=True, page_size=16, skip_tokenizer_init=True,
                  max_total_tokens=1024, dtype="float32", log_level="error", disaggregation_shared_secret="pd",
                  disaggregation_transfer_port=0, disaggregation_side_channel_port=0)
    prefill = Engine(**common, disaggregation_mode="prefill", disaggregation_bootstrap_port=port)
    monkeypatch.delenv("DISAGG_LAUNCH_BOOTSTRAP")
    decode = Engine(**common, disaggregation_mode="decode", disaggregation_bootstrap_url=f"http://127.0.0.1:{port}",
                    disaggregation_decode_watchdog_seconds=30.0)
    try:
        assert prefill.scheduler.disagg_bootstrap_server.url == f"http://127.0.0.1:{port}"
        assert prefill.scheduler.server_args.disaggregation_bootstrap_url == f"http://127.0.0.1:{port}"
        wd = decode.scheduler.disagg_decode_watchdog
        assert wd.timeout == 30.0 and wd._thread.is_alive() and wd.stalls == 0
        sp = {"temperature": 0.0, "max_new_tokens": 4, "ignore_eos": True}
        res = {}
        ts = [threading.Thread(target=lambda: res.update(d=decode.generate(input_ids=list(range(5, 45)), sampling_params=sp,
                                                                          bootstrap_room=7))),
              threading.Thread(target=lambda: res.update(p=prefill.generate(input_ids=list(range(5, 45)), sampling_params=sp,
                                                                           bootstrap_room=7)))]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=120)
        assert len(res["d"]["output_ids"]) == 4 and res["d"]["output_ids"][0] == res["p"]["output_ids"][0]
    finally:
        shutdown_disaggregation(prefill.scheduler, 1)
        shutdown_disaggregation(decode.scheduler, 1)
        prefill.shutdown()
        decode.shutdown()
    assert not decode.scheduler.disagg_decode_watchdog._thread.is_alive()
    assert prefill.scheduler.disagg_bootstrap_server is None


def test_in_node_pd_front_door_matches_single_engine(tmp_path):
    """`--pd-disaggregation`: one `Engine(...)` call builds prefill and decode engines on slices of the node's
    devices with an embedded registry; requests fan out to a prefill and a decode engine and the answers are those
    of a monolithic engine (reference: the in-process P/D split of `pathways_pd.py` / `pathways_scheduler.py`)."""
    from sglang_jax_b200.disaggregation.local_pd import LocalPDEngine
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import write_tiny_qwen3_checkpoint
    ckpt = write_tiny_qwen3_checkpoint(str(tmp_path / "m"))
    rng = np.random.RandomState(3)
    prompts = [rng.randint(5, 1000, size=n).tolist() for n in (33, 70, 18, 51)]
    sp = {"temperature": 0.0, "max_new_tokens": 6, "ignore_eos": True}
    common = dict(model_path=ckpt, device="cpu", enable_single_process=True, page_size=16, skip_tokenizer_init=True,
                  max_total_tokens=2048, dtype="float32", log_level="error")
    ps.reset_state()
    plain = Engine(**common)
    try:
        want = [o["output_ids"] for o in plain.generate(input_ids=prompts, sampling_params=sp)]
    finally:
        plain.shutdown()
    ps.reset_state()
    eng = Engine(**common, pd_disaggregation="local", pd_num_prefill=1, pd_num_decode=2,
                 disaggregation_bootstrap_port=get_free_port(), chunked_prefill_size=32)
    try:
        assert isinstance(eng, LocalPDEngine) and len(eng.prefill) == 1 and len(eng.decode) == 2
        assert [e.server_args.device_indexes for e in eng.engines()] == [[0], [1], [2]]
        assert eng.prefill[0].server_args.disaggregation_mode == "prefill"
        outs = eng.generate(input_ids=prompts, sampling_params=sp)
        assert [o["output_ids"] for o in outs] == want
        assert sorted(o["meta_info"]["pd_decode_engine"] for o in outs) == [0, 0, 1, 1]      # spread over both
        one = eng.generate(input_ids=prompts[0], sampling_params=sp)
        assert one["output_ids"] == want[0] and one["meta_info"]["bootstrap_room"] == 5
        # concurrent callers overlap on the same engines
        res = {}
        ts = [threading.Thread(target=lambda i=i: res.update({i: eng.generate(input_ids=prompts[i], sampling_params=sp)}))
              for i in range(4)]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=120)
        assert [res[i]["output_ids"] for i in range(4)] == want
        info = eng.get_server_info()
        assert info["pd_routed"]["prefill"] == [9] and sum(info["pd_routed"]["decode"]) == 9
        # the HTTP surface `launch_server --pd-disaggregation` exposes
        from fastapi.testclient import TestClient
        from sglang_jax_b200.disaggregation.local_pd import build_pd_app
        with TestClient(build_pd_app(eng)) as client:
            assert client.get("/health").json() == {"status": "ok", "prefill": 1, "decode": 2}
            r = client.post("/generate", json={"input_ids": prompts[1], "sampling_params": sp})
            assert r.status_code == 200 and r.json()["output_ids"] == want[1]
            r = client.post("/generate", json={"input_ids": prompts[:2], "sampling_params": sp})
            assert [o["output_ids"] for o in r.json()] == want[:2]
            assert client.post("/generate", json={"input_ids": prompts[0], "stream": True}).status_code == 400
            assert client.get("/get_server_info").json()["pd_routed"]["prefill"] == [12]
        time.sleep(0.2)
        for e in eng.engines():
            e.scheduler.check_memory()
    finally:
        eng.shutdown()
    with pytest.raises(ValueError, match="needs 3 devices"):
        Engine(**common, pd_disaggregation="local", pd_num_decode=2, device_indexes=[0, 1])
