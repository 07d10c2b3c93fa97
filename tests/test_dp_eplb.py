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
