"""Speculative decoding on CPU: whatever the draft proposes, greedy output must equal the
plain engine's output token for token (reference test strategy:
`python/sgl_jax/test/speculative/`)."""

import numpy as np
import pytest
import torch

from sglang_jax_b200.speculative.eagle_util import (build_tree, tree_speculative_sampling_target_only,
                                                    verify_tree_greedy)


def test_build_tree_and_greedy_verify():
    # k=2, S=2: depth-1 candidates ids 1,2; depth-2 candidates ids 3..6 (parents 1,1,2,2)
    tok = torch.tensor([[10, 11, 20, 21, 22, 23]])
    score = torch.tensor([[0.6, 0.4, 0.5, 0.1, 0.3, 0.1]])
    parent = torch.tensor([[0, 0, 1, 1, 2, 2]])
    tokens, par, depth, mask, sel = build_tree(torch.tensor([7]), tok, score, parent, 5, 2)
    assert tokens.tolist() == [[7, 10, 11, 20, 22]]
    assert par.tolist() == [[-1, 0, 0, 1, 2]]
    assert depth.tolist() == [[0, 1, 1, 2, 2]]
    m = mask[0].int().tolist()
    assert m[3] == [1, 1, 0, 1, 0] and m[4] == [1, 0, 1, 0, 1]
    # target prefers 11 after root, then 22 after 11, then 99
    target = torch.tensor([[11, 0, 22, 0, 99]])
    acc, path, bonus = verify_tree_greedy(tokens, par, target, 2)
    assert acc.tolist() == [2] and path.tolist() == [[0, 2, 4]] and bonus.tolist() == [99]
    # mismatch at the first level
    acc, path, bonus = verify_tree_greedy(tokens, par, torch.tensor([[5, 0, 0, 0, 0]]), 2)
    assert acc.tolist() == [0] and bonus.tolist() == [5]


def test_stochastic_verify_matches_target_distribution():
    torch.manual_seed(0)
    V = 6
    p_root = torch.tensor([0.05, 0.4, 0.3, 0.15, 0.05, 0.05])
    # chain-free tree: two children of the root proposing tokens 1 and 2
    tokens = torch.tensor([[0, 1, 2]])
    parent = torch.tensor([[-1, 0, 0]])
    N = 20000
    probs = torch.zeros(N, 3, V)
    probs[:, 0] = p_root
    probs[:, 1] = torch.tensor([1.0, 0, 0, 0, 0, 0])
    probs[:, 2] = torch.tensor([1.0, 0, 0, 0, 0, 0])
    coins = torch.rand(N, 2)
    final = torch.rand(N)
    acc, path, bonus = tree_speculative_sampling_target_only(tokens.expand(N, -1), parent.expand(N, -1), probs,
                                                             coins, final, 1)
    first = torch.where(acc > 0, tokens[0][path[:, 1].clamp_min(0)], bonus)
    freq = torch.bincount(first, minlength=V).float() / N
    assert torch.allclose(freq, p_root, atol=0.015), freq


def _ckpt(path, seed, **over):
    from sglang_jax_b200.utils.tiny_models import TINY_QWEN3, write_tiny_qwen3_checkpoint
    return write_tiny_qwen3_checkpoint(str(path), seed=seed, config=dict(TINY_QWEN3, **over))


def _fresh():
    from sglang_jax_b200.parallel import state as ps
    ps.reset_state()


@pytest.mark.parametrize("topk,steps,ndraft,page", [(1, 3, 4, 1), (1, 3, 4, 4), (2, 3, 6, 1), (3, 2, 5, 4)])
def test_standalone_matches_plain_greedy(tmp_path, topk, steps, ndraft, page):
    from sglang_jax_b200.entrypoints.engine import Engine
    target = _ckpt(tmp_path / "target", 0)
    draft = _ckpt(tmp_path / "draft", 1, num_hidden_layers=1)
    prompts = [[3, 17, 42, 9, 5, 11, 8], [4, 4, 19, 23], [7] * 11]
    sp = {"temperature": 0.0, "max_new_tokens": 24, "ignore_eos": True}
    common = dict(model_path=target, device="cpu", enable_single_process=True, page_size=page,
                  skip_tokenizer_init=True, max_total_tokens=2048, chunked_prefill_size=16 if page > 1 else 8,
                  random_seed=0, dtype="float32", log_level="error")
    _fresh()
    plain = Engine(**common)
    try:
        ref = [o["output_ids"] for o in plain.generate(input_ids=prompts, sampling_params=sp)]
    finally:
        plain.shutdown()
    _fresh()
    spec = Engine(**common, speculative_algorithm="STANDALONE", speculative_draft_model_path=draft,
                  speculative_num_steps=steps, speculative_eagle_topk=topk, speculative_num_draft_tokens=ndraft)
    try:
        outs = spec.generate(input_ids=prompts, sampling_params=sp)
        got = [o["output_ids"] for o in outs]
        assert got == ref
        assert all(o["meta_info"].get("spec_verify_ct", 0) > 0 for o in outs)
        # nothing leaked: all KV slots are back once the requests are done
        spec.flush_cache()
    finally:
        spec.shutdown()


def test_self_draft_accepts_everything(tmp_path):
    """With the target itself as the (shifted-input) draft the acceptance rate is high but
    the output is still exactly the plain one."""
    from sglang_jax_b200.entrypoints.engine import Engine
    target = _ckpt(tmp_path / "target", 0)
    prompts = [[3, 17, 42, 9, 5, 11, 8, 2, 2, 6]]
    sp = {"temperature": 0.0, "max_new_tokens": 16, "ignore_eos": True}
    common = dict(model_path=target, device="cpu", enable_single_process=True, page_size=1,
                  skip_tokenizer_init=True, max_total_tokens=1024, random_seed=0, dtype="float32",
                  log_level="error")
    _fresh()
    plain = Engine(**common)
    try:
        ref = plain.generate(input_ids=prompts, sampling_params=sp)[0]["output_ids"]
    finally:
        plain.shutdown()
    _fresh()
    spec = Engine(**common, speculative_algorithm="STANDALONE", speculative_draft_model_path=target,
                  speculative_num_steps=3, speculative_eagle_topk=1, speculative_num_draft_tokens=4)
    try:
        out = spec.generate(input_ids=prompts, sampling_params=sp)[0]
        assert out["output_ids"] == ref
    finally:
        spec.shutdown()


def _plain_vs_spec(target, prompts, sp, spec_kw, page=1, **extra):
    from sglang_jax_b200.entrypoints.engine import Engine
    common = dict(model_path=target, device="cpu", enable_single_process=True, page_size=page,
                  skip_tokenizer_init=True, max_total_tokens=2048, random_seed=0, dtype="float32",
                  log_level="error", **extra)
    _fresh()
    plain = Engine(**common)
    try:
        ref = [o["output_ids"] for o in plain.generate(input_ids=prompts, sampling_params=sp)]
    finally:
        plain.shutdown()
    _fresh()
    spec = Engine(**common, **spec_kw)
    try:
        outs = spec.generate(input_ids=prompts, sampling_params=sp)
        spec.scheduler.check_memory()
    finally:
        spec.shutdown()
    return ref, outs


@pytest.mark.parametrize("kind,dv,topk", [("eagle", None, 1), ("eagle", None, 3), ("eagle3", None, 2), ("eagle3", 256, 1)])
def test_eagle_heads_keep_greedy_output(tmp_path, kind, dv, topk):
    from sglang_jax_b200.utils.tiny_models import write_tiny_eagle_checkpoint
    target = _ckpt(tmp_path / "target", 0)
    draft = write_tiny_eagle_checkpoint(str(tmp_path / "draft"), kind=kind, draft_vocab_size=dv)
    prompts = [[3, 17, 42, 9, 5, 11, 8], [4, 4, 19, 23, 99, 100, 101, 102, 103]]
    sp = {"temperature": 0.0, "max_new_tokens": 20, "ignore_eos": True}
    ref, outs = _plain_vs_spec(target, prompts, sp, dict(
        speculative_algorithm="EAGLE3" if kind == "eagle3" else "EAGLE", speculative_draft_model_path=draft,
        speculative_num_steps=3, speculative_eagle_topk=topk, speculative_num_draft_tokens=4 if topk == 1 else 6),
        page=4 if topk == 1 else 1, chunked_prefill_size=8)
    assert [o["output_ids"] for o in outs] == ref


@pytest.mark.parametrize("layers", [1, 2])
def test_nextn_mtp_keeps_greedy_output(tmp_path, layers):
    from sglang_jax_b200.utils.tiny_models import write_tiny_mimo_checkpoint
    target = write_tiny_mimo_checkpoint(str(tmp_path / "mimo"), num_mtp_layers=layers)
    prompts = [[3, 17, 42, 9, 5, 11, 8], [4, 4, 19, 23]]
    sp = {"temperature": 0.0, "max_new_tokens": 16, "ignore_eos": True}
    ref, outs = _plain_vs_spec(target, prompts, sp, dict(
        speculative_algorithm="NEXTN", speculative_num_steps=3, speculative_eagle_topk=1,
        speculative_num_draft_tokens=4), page=4)
    assert [o["output_ids"] for o in outs] == ref


def test_stop_token_inside_accepted_run(tmp_path):
    """A stop token in the middle of an accepted run ends the request there."""
    target = _ckpt(tmp_path / "target", 0)
    prompts = [[3, 17, 42, 9, 5, 11, 8, 2, 2, 6]]
    base = {"temperature": 0.0, "max_new_tokens": 16, "ignore_eos": True}
    ref, _ = _plain_vs_spec(target, prompts, base, dict(
        speculative_algorithm="STANDALONE", speculative_draft_model_path=target, speculative_num_steps=3,
        speculative_eagle_topk=1, speculative_num_draft_tokens=4))
    stop = ref[0][5]
    first = ref[0].index(stop)
    sp = dict(base, ignore_eos=False, stop_token_ids=[stop])
    ref2, outs = _plain_vs_spec(target, prompts, sp, dict(
        speculative_algorithm="STANDALONE", speculative_draft_model_path=target, speculative_num_steps=3,
        speculative_eagle_topk=1, speculative_num_draft_tokens=4))
    assert ref2[0] == ref[0][:first + 1]
    assert outs[0]["output_ids"] == ref2[0]


@pytest.mark.parametrize("page,block", [(1, 4), (4, 3)])
def test_dflash_block_draft_keeps_greedy_output(tmp_path, page, block):
    from sglang_jax_b200.utils.tiny_models import write_tiny_dflash_checkpoint
    target = _ckpt(tmp_path / "target", 0)
    draft = write_tiny_dflash_checkpoint(str(tmp_path / "draft"), block_size=block)
    prompts = [[3, 17, 42, 9, 5, 11, 8], [4, 4, 19, 23, 99, 100, 101, 102, 103]]
    sp = {"temperature": 0.0, "max_new_tokens": 16, "ignore_eos": True}
    ref, outs = _plain_vs_spec(target, prompts, sp, dict(
        speculative_algorithm="DFLASH", speculative_draft_model_path=draft, speculative_num_draft_tokens=block),
        page=page, chunked_prefill_size=8)
    assert [o["output_ids"] for o in outs] == ref


def _spec_tp_rank(rank, world, port, target, draft, algo, q):
    import os
    import sys
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.server_args import ServerArgs
    torch.set_num_threads(2)
    ps.init_distributed(rank, world, "cpu", init_method=f"tcp://127.0.0.1:{port}", timeout_s=120)
    sa = ServerArgs(model_path=target, device="cpu", dtype="float32", page_size=4, skip_tokenizer_init=True,
                    max_total_tokens=2048, enable_single_process=True, tp_size=world, log_level="error",
                    watchdog_timeout=0, chunked_prefill_size=16, speculative_algorithm=algo,
                    speculative_draft_model_path=draft, speculative_num_steps=3, speculative_eagle_topk=2,
                    speculative_num_draft_tokens=6)
    if rank != 0:
        from sglang_jax_b200.managers.tp_worker import run_tp_follower
        run_tp_follower(sa)
    else:
        from sglang_jax_b200 import Engine
        eng = Engine(server_args=sa)
        prompts = [[3, 17, 42, 9, 5, 11, 8], [4, 4, 19, 23, 99, 100, 101, 102, 103] * 3]
        outs = eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 16, "temperature": 0.0,
                                                                 "ignore_eos": True})
        sampled = eng.generate(input_ids=prompts[:1], sampling_params={"max_new_tokens": 8, "temperature": 0.9,
                                                                       "ignore_eos": True})
        q.put(([o["output_ids"] for o in outs], len(sampled[0]["output_ids"])))
        eng.shutdown()
    ps.destroy()


@pytest.mark.parametrize("algo", ["EAGLE", "STANDALONE"])
def test_speculative_under_tensor_parallel_2(tmp_path, algo):
    """Follower ranks mirror every draft / verify forward from the host inputs rank 0 ships."""
    import torch.multiprocessing as mp
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.utils.common import get_free_port
    from sglang_jax_b200.utils.tiny_models import write_tiny_eagle_checkpoint
    target = _ckpt(tmp_path / "target", 0)
    draft = write_tiny_eagle_checkpoint(str(tmp_path / "draft")) if algo == "EAGLE" else \
        _ckpt(tmp_path / "draft", 1, num_hidden_layers=1)
    prompts = [[3, 17, 42, 9, 5, 11, 8], [4, 4, 19, 23, 99, 100, 101, 102, 103] * 3]
    _fresh()
    plain = Engine(model_path=target, device="cpu", enable_single_process=True, page_size=4, skip_tokenizer_init=True,
                   max_total_tokens=2048, dtype="float32", log_level="error")
    try:
        want = [o["output_ids"] for o in plain.generate(input_ids=prompts, sampling_params={
            "max_new_tokens": 16, "temperature": 0.0, "ignore_eos": True})]
    finally:
        plain.shutdown()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = get_free_port()
    procs = [ctx.Process(target=_spec_tp_rank, args=(r, 2, port, target, draft, algo, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        got, n_sampled = q.get(timeout=300)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    assert got == want and n_sampled == 8


def test_mimo_v2_nextn_swa_draft_keeps_greedy_output(tmp_path):
    """Random-weight MiMo-V2 target (hybrid SWA + MoE) with its sliding-window MTP layers as draft."""
    import json
    cfg = dict(architectures=["MiMoV2FlashForCausalLM"], model_type="mimo_v2_flash", hidden_size=64,
               intermediate_size=96, moe_intermediate_size=32, num_hidden_layers=3, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, v_head_dim=8, swa_num_attention_heads=4, swa_num_key_value_heads=4,
               swa_head_dim=16, swa_v_head_dim=8, swa_rope_theta=10000.0, rope_theta=1000000.0,
               sliding_window_size=16, hybrid_layer_pattern=[0, 1, 0], moe_layer_freq=[0, 1, 1],
               add_swa_attention_sink_bias=True, n_routed_experts=4, num_experts_per_tok=2, scoring_func="sigmoid",
               topk_method="noaux_tc", norm_topk_prob=True, layernorm_epsilon=1e-5, vocab_size=256,
               max_position_embeddings=512, tie_word_embeddings=False, num_nextn_predict_layers=2,
               torch_dtype="float32")
    path = tmp_path / "mimo2"
    path.mkdir()
    (path / "config.json").write_text(json.dumps(cfg))
    prompts = [list(range(3, 40)), [4, 4, 19, 23]]
    sp = {"temperature": 0.0, "max_new_tokens": 16, "ignore_eos": True}
    ref, outs = _plain_vs_spec(str(path), prompts, sp, dict(
        speculative_algorithm="NEXTN", speculative_num_steps=3, speculative_eagle_topk=1,
        speculative_num_draft_tokens=4), page=4, load_format="dummy")
    assert [o["output_ids"] for o in outs] == ref
