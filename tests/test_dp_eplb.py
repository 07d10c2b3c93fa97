import pytest
import numpy as np
import torch

from sglang_jax_b200.eplb.expert_location import ExpertLocation, balanced_packing, rebalance, replicate_experts
from sglang_jax_b200.managers.dp_schedule_policy import DPRankAssignment, DPRankLoad, create_dp_schedule_policy
from sglang_jax_b200.mem_cache.radix_cache import RadixCache, RadixKey


class R:
    def __init__(self, ids, extra_key=None):
        self.origin_input_ids = ids
        self.extra_key = extra_key


def test_dp_policies():
    loads = [DPRankLoad(3, 2, 500, 1000), DPRankLoad(1, 0, 0, 100), DPRankLoad(2, 2, 50, 10)]
    rr = create_dp_schedule_policy("round_robin", 3)
    assert [rr.select(None, loads) for _ in range(4)] == [0, 1, 2, 0]
    assert create_dp_schedule_policy("min_running_queue", 3).select(None, loads) == 1
    assert create_dp_schedule_policy("shape_aware", 3).select(None, loads) == 1
    cache = RadixCache(None, None, 1)
    cache.insert(RadixKey(list(range(100)), None, 2), np.arange(100))
    ca = create_dp_schedule_policy("cache_aware", 3)
    assert ca.select(R(list(range(80)) + [999]), loads, cache) == 2       # long cached prefix on rank 2
    assert ca.select(R([7, 8, 9, 10]), loads, cache) == 1                 # no match -> lightest
    heavy = [DPRankLoad(1, 0), DPRankLoad(1, 0), DPRankLoad(100, 50)]
    assert ca.select(R(list(range(80)) + [999]), heavy, cache) == 0       # imbalance guard
    a = DPRankAssignment(3)
    assert a.assign("x", 2) == 2 and a.assign("x", 0) == 2 and a.counts() == [0, 0, 1]
    a.release("x")
    assert a.get("x") is None


def test_eplb_replication_and_packing():
    load = np.array([100, 10, 10, 10, 50, 10, 10, 10])
    phy2log, cnt = replicate_experts(load.astype(float), 12)
    assert cnt[0] >= 3 and cnt[4] >= 2 and cnt.sum() == 12
    pack = balanced_packing(np.array([9, 1, 8, 2, 7, 3, 6, 4], dtype=float), 4)
    sums = [sum(w for w, p in zip([9, 1, 8, 2, 7, 3, 6, 4], pack) if p == q) for q in range(4)]
    assert max(sums) - min(sums) <= 2
    m = rebalance(load, 12, 4)
    assert len(m) == 12 and set(m.tolist()) == set(range(8))
    loc = ExpertLocation.from_load(load, ep_size=4, num_redundant=4)
    ids = torch.tensor([[0, 4], [0, 1], [0, 7], [0, 4]], dtype=torch.int32)
    phy = loc.logical_to_physical(ids)
    assert (torch.as_tensor(loc.phy2log)[phy.long()] == ids.long()).all()
    assert len(set(phy[:, 0].tolist())) > 1          # the hot expert is spread over replicas
    w = torch.arange(8).float().view(8, 1)
    assert loc.physical_weights(w).view(-1).tolist() == [float(x) for x in loc.phy2log]


def test_eplb_hierarchical_keeps_groups_on_nodes_and_balances_ranks():
    """Node-aware placement for group-limited routing: whole expert groups stay on one node, spare slots go to the
    node's hot experts, ranks inside a node carry similar load; `auto` picks it when the groups divide over nodes."""
    from sglang_jax_b200.eplb.expert_location import rebalance_experts, rebalance_hierarchical
    rng = np.random.RandomState(0)
    E, groups, nodes, ranks, phy = 32, 4, 2, 8, 40
    load = rng.gamma(0.6, 100.0, size=E) + 1
    m = rebalance_hierarchical(load, phy, groups, nodes, ranks)
    assert len(m) == phy and set(m.tolist()) == set(range(E))
    per_node = phy // nodes
    node_of_group = {}
    for p, e in enumerate(m.tolist()):
        assert node_of_group.setdefault(e // (E // groups), p // per_node) == p // per_node     # a group lives on one node
    cnt = np.bincount(m, minlength=E)
    slots = phy // ranks
    rank_load = np.array([sum(load[e] / cnt[e] for e in m[r * slots:(r + 1) * slots]) for r in range(ranks)])
    naive = load.reshape(ranks, -1).sum(1)
    assert rank_load.max() / rank_load.mean() < naive.max() / naive.mean()
    assert np.array_equal(rebalance_experts(load, phy, ranks, groups, nodes, "auto"), m)
    flat = rebalance_experts(load, phy, ranks, groups, 1, "auto")                # one node: the global algorithm
    assert np.array_equal(flat, rebalance(load, phy, ranks))
    loc = ExpertLocation.from_load(load, ep_size=ranks, num_redundant=phy - E, num_groups=groups, num_nodes=nodes)
    assert np.array_equal(loc.phy2log, m)
    with pytest.raises(ValueError):
        rebalance_hierarchical(load, phy, 3, 2, ranks)


def test_data_parallel_replicas_route_and_match_single_engine(tmp_path):
    """dp_size=2: two replicas behind the router produce exactly the single-engine outputs, the
    router spreads the requests, and a pinned `dp_rank` is honoured."""
    import numpy as np
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.managers.data_parallel_controller import DataParallelEngine
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import write_tiny_qwen3_checkpoint
    ckpt = write_tiny_qwen3_checkpoint(str(tmp_path / "m"))
    rng = np.random.RandomState(0)
    prompts = [rng.randint(5, 1000, size=n).tolist() for n in (12, 30, 7, 19, 25, 9)]
    sp = {"temperature": 0.0, "max_new_tokens": 6, "ignore_eos": True}
    common = dict(model_path=ckpt, device="cpu", enable_single_process=True, page_size=4, skip_tokenizer_init=True,
                  max_total_tokens=2048, dtype="float32", log_level="error")
    ps.reset_state()
    one = Engine(**common)
    try:
        want = [o["output_ids"] for o in one.generate(input_ids=prompts, sampling_params=sp)]
    finally:
        one.shutdown()
    ps.reset_state()
    eng = Engine(**common, dp_size=2, tp_size=2, dp_schedule_policy="round_robin")
    try:
        assert isinstance(eng, DataParallelEngine) and len(eng.replicas) == 2
        outs = eng.generate(input_ids=prompts, sampling_params=sp)
        assert [o["output_ids"] for o in outs] == want
        assert [o["meta_info"]["dp_rank"] for o in outs] == [0, 1, 0, 1, 0, 1] and eng.routed == [3, 3]
        pinned = eng.generate(input_ids=prompts[:2], sampling_params=sp, dp_rank=1)
        assert [o["meta_info"]["dp_rank"] for o in pinned] == [1, 1]
        assert eng.generate(input_ids=prompts[0], sampling_params=sp)["output_ids"] == want[0]
        assert len(eng.get_server_info()["internal_states"]) == 2
    finally:
        eng.shutdown()


# ------------------------------------------------------------------------------------------
# routed-expert capture, hit-count recorder and redundant experts inside a running engine
def _tiny_moe(tmp_path):
    import torch
    from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM
    from test_models_cpu import _init, _save
    cfg = dict(hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, rope_theta=1e6,
               vocab_size=512, num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1,
               mlp_only_layers=[], tie_word_embeddings=False, max_position_embeddings=512)
    hf = _init(Qwen3MoeForCausalLM(Qwen3MoeConfig(**cfg)))
    return hf, _save(str(tmp_path / "moe"), hf, cfg, "Qwen3MoeForCausalLM", "qwen3_moe")


def test_engine_returns_routed_experts_and_records_expert_load(tmp_path):
    import numpy as np
    import torch
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    hf, path = _tiny_moe(tmp_path)
    dump = str(tmp_path / "load.npy")
    prompts = [list(range(5, 40)), [9, 8, 7, 6, 5, 4, 3] * 3]
    ps.reset_state()
    eng = Engine(model_path=path, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                 max_total_tokens=4096, enable_single_process=True, enable_return_routed_experts=True,
                 enable_expert_distribution_recorder=True, expert_distribution_recorder_buffer_size=1,
                 expert_distribution_recorder_output_file=dump, disable_radix_cache=True)
    try:
        outs = eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 4, "temperature": 0,
                                                                "ignore_eos": True}, return_routed_experts=True)
        plain = eng.generate(input_ids=prompts[:1], sampling_params={"max_new_tokens": 2, "temperature": 0})
    finally:
        eng.shutdown()
    assert "routed_experts" not in plain[0]["meta_info"] or not plain[0]["meta_info"]["routed_experts"]
    for ids, o in zip(prompts, outs):
        got = np.asarray(o["meta_info"]["routed_experts"])          # [tokens, layers, top_k]
        assert got.shape == (len(ids) + 4 - 1, 2, 2), got.shape
        # the router's choice for the prompt tokens is the HF model's
        with torch.no_grad():
            ref = hf(torch.tensor([ids]), output_router_logits=True).router_logits
        for layer in range(2):
            want = torch.topk(ref[layer].float(), 2, dim=-1).indices.sort(-1).values.numpy()
            assert np.array_equal(np.sort(got[: len(ids), layer], -1), want), layer
    load = np.load(dump)
    assert load.shape == (2, 8) and load.sum() >= 2 * 2 * sum(len(p) for p in prompts)
    # --enable-expert-balance-debug through the engine: segments of two decode steps land in the CSV
    import csv
    bal = str(tmp_path / "balance.csv")
    ps.reset_state()
    eng = Engine(model_path=path, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                 max_total_tokens=4096, enable_single_process=True, enable_expert_balance_debug=True,
                 expert_balance_segment_counter=2, expert_balance_output_file=bal, disable_radix_cache=True)
    try:
        eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 6, "temperature": 0, "ignore_eos": True})
    finally:
        eng.shutdown()
    rows = list(csv.DictReader(open(bal)))
    assert len(rows) >= 4 and {r["layer"] for r in rows} == {"0", "1"} and rows[0]["topk"] == "2"
    assert all(int(r["total_assignments"]) > 0 and len(r["experts_count"].split()) == 8 for r in rows)


def _ep_rank(rank, world, port, path, q, redundant, load_file, moe_backend="epmoe"):
    import os
    import sys
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.server_args import ServerArgs
    torch.set_num_threads(2)
    ps.init_distributed(rank, world, "cpu", 1, world, init_method=f"tcp://127.0.0.1:{port}", timeout_s=120)
    sa = ServerArgs(model_path=path, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                    max_total_tokens=4096, enable_single_process=True, tp_size=world, ep_size=world,
                    ep_num_redundant_experts=redundant, init_expert_location=load_file or "trivial",
                    log_level="error", watchdog_timeout=0, moe_backend=moe_backend)
    if rank != 0:
        from sglang_jax_b200.managers.tp_worker import run_tp_follower
        run_tp_follower(sa)
    else:
        from sglang_jax_b200 import Engine
        from sglang_jax_b200.layers.moe import FusedMoE
        eng = Engine(server_args=sa)
        moes = [m for m in eng.scheduler.tp_worker.model_runner.model.modules() if isinstance(m, FusedMoE)]
        info = [(m.num_experts, m.num_local_experts,
                 m.expert_location.phy2log.tolist() if m.expert_location is not None else None) for m in moes]
        outs = eng.generate(input_ids=[list(range(5, 40)), [9, 8, 7, 6, 5, 4, 3] * 5],
                            sampling_params={"max_new_tokens": 8, "temperature": 0.0, "ignore_eos": True})
        from sglang_jax_b200.layers import fused_ep_moe
        assert (fused_ep_moe.CALLS > 0) == (moe_backend == "fused")
        q.put(([o["output_ids"] for o in outs], info))
        eng.shutdown()
    ps.destroy()


def test_redundant_experts_keep_outputs_and_follow_recorded_load(tmp_path):
    """EP2 with two redundant expert slots: replicas hold copies of their logical expert, tokens are dealt over
    the replicas, outputs equal the single-GPU HF model; a recorded load file steers which experts are doubled."""
    import numpy as np
    import torch.multiprocessing as mp
    from test_models_cpu import _hf_generate
    from sglang_jax_b200.utils.common import get_free_port
    hf, path = _tiny_moe(tmp_path)
    want = _hf_generate(hf, [list(range(5, 40)), [9, 8, 7, 6, 5, 4, 3] * 5], n=8)
    load = np.ones((2, 8))
    load[:, 5] = 50
    load[:, 2] = 30          # experts 5 and 2 are the hot ones
    load_file = str(tmp_path / "load.npy")
    np.save(load_file, load)
    for lf in (None, load_file):
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = get_free_port()
        procs = [ctx.Process(target=_ep_rank, args=(r, 2, port, path, q, 2, lf)) for r in range(2)]
        for p in procs:
            p.start()
        try:
            outs, info = q.get(timeout=300)
        finally:
            for p in procs:
                p.join(timeout=60)
                if p.is_alive():
                    p.kill()
        assert outs == want
        for n_phys, n_local, phy2log in info:
            assert n_phys == 10 and n_local == 5 and sorted(set(phy2log)) == list(range(8))
            if lf:
                assert sorted(phy2log.count(e) for e in (5, 2)) == [2, 2]


@pytest.mark.parametrize("world,redundant", [(2, 0), (4, 0), (2, 2)])
def test_token_all_to_all_moe_matches_hf(tmp_path, world, redundant):
    """`--moe-backend fused`: tokens stay sharded over the expert-parallel ranks, (token, expert) rows travel to the
    expert's rank and back (here through the process group's all-to-all, the oracle of the NVLink kernels)."""
    import torch.multiprocessing as mp
    from test_models_cpu import _hf_generate
    from sglang_jax_b200.utils.common import get_free_port
    hf, path = _tiny_moe(tmp_path)
    prompts = [list(range(5, 40)), [9, 8, 7, 6, 5, 4, 3] * 5]
    want = _hf_generate(hf, prompts, n=8)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = get_free_port()
    procs = [ctx.Process(target=_ep_rank, args=(r, world, port, path, q, redundant, None, "fused")) for r in range(world)]
    for p in procs:
        p.start()
    try:
        outs, _ = q.get(timeout=300)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    assert outs == want


def test_expert_balance_debug_writes_segments_and_static_dispatch(tmp_path):
    """`--enable-expert-balance-debug`: one CSV row per layer and segment of decode steps with the hit counts and the
    imbalance over experts / expert-parallel ranks; `--ep-dispatch-algorithm static` keeps a logical expert's tokens
    on its first replica."""
    import csv
    from sglang_jax_b200.eplb.expert_location import ExpertBalanceAnalyzer
    out = tmp_path / "bal" / "balance.csv"
    a = ExpertBalanceAnalyzer(num_layers=2, num_experts=8, topk=2, ep_size=4, segment_counter=3, output_file=str(out))
    ids = torch.tensor([[0, 1], [0, 2], [0, 3], [0, 7]])
    for stepno in range(7):
        a.record(0, ids)
        if stepno % 2 == 0:
            a.record(1, ids[:, :1] + 4)
        a.step(is_decode=True)
        a.step(is_decode=False)                 # prefill steps do not advance a segment
    rows = list(csv.DictReader(open(out)))
    assert len(rows) == 4 and [r["segment_idx"] for r in rows] == ["0", "0", "1", "1"]
    first = rows[0]
    assert first["layer"] == "0" and first["total_assignments"] == "24" and first["segment_decode_steps"] == "3"
    assert first["experts_count"].split()[0] == "12" and float(first["max_over_mean_expert"]) == 4.0
    assert float(first["max_over_mean_device"]) == pytest.approx(15 / 6, rel=1e-3)       # ranks hold experts (0,1), (2,3), ...
    assert a.segment_idx == 2 and a.decode_steps == 1
    loc = ExpertLocation(4, 2, 2, phy2log=np.array([0, 1, 0, 2, 3, 0]))
    hot = torch.zeros(6, 1, dtype=torch.int32)
    assert len(set(loc.logical_to_physical(hot).flatten().tolist())) == 3                # dealt over the replicas
    loc.dispatch_algorithm = "static"
    assert set(loc.logical_to_physical(hot).flatten().tolist()) == {0}
