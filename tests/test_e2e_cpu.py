"""End-to-end plumbing on CPU in fp32: the tiny Qwen3 config (2 layers, hidden 256, 4q/2kv heads,
head_dim 64 + q/k norm, FFN 512, vocab 1024, tied embeddings, page 16, radix cache on, 8 requests of
which 4 share a 64-token prefix, greedy, 32 new tokens) must reproduce HF transformers' Qwen3 tokens
exactly, independent of radix cache, chunking, overlap scheduling and tensor parallelism."""

import os
import sys

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
])
def test_outputs_invariant_to_scheduling_options(ckpt, oracle, kw):
    outs, _, _ = run_engine(ckpt, **kw)
    assert outs == oracle


def test_prefix_cache_hits_are_reported(ckpt):
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    ps.reset_state()
    eng = Engine(model_path=ckpt, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                 max_total_tokens=8192, enable_single_process=True)
    try:
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
