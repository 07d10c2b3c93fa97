"""End-to-end numerics on the GPU: the model forward with the sm_100a kernels against the same
forward with the plain-PyTorch ops, eager vs CUDA-graph decode, and the engine API."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny_path():
    from sglang_jax_b200.utils.tiny_models import TINY_QWEN3, write_tiny_qwen3_checkpoint
    cfg = dict(TINY_QWEN3, head_dim=128, num_attention_heads=8, num_key_value_heads=2, hidden_size=1024,
               intermediate_size=2048, num_hidden_layers=3, torch_dtype="bfloat16", tie_word_embeddings=False)
    return write_tiny_qwen3_checkpoint("/tmp/sglb200_test_qwen3_gpu", config=cfg, dtype=torch.bfloat16)


def _runner(path, **kw):
    from sglang_jax_b200.configs.model_config import ModelConfig
    from sglang_jax_b200.model_executor.model_runner import ModelRunner
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.server_args import ServerArgs
    ps.reset_state()
    ps.init_distributed(0, 1, "cuda")
    # these tests compare graph replays with eager steps token for token: keep the measured GEMM plan among this
    # library's own kernels (a library GEMM may pick another algorithm, hence another summation order, under capture)
    import os
    os.environ["SGLB_GEMM_PLAN_LIBRARY"] = "0"
    sa = ServerArgs(model_path=path, device="cuda", dtype="bfloat16", page_size=16, skip_tokenizer_init=True,
                    max_total_tokens=8192, max_running_requests=16, disable_overlap_schedule=True, **kw)
    return ModelRunner(ModelConfig.from_server_args(sa), sa), sa


def _extend_batch(runner, lens, prefix=None, seed=0):
    from sglang_jax_b200.managers.schedule_batch import ForwardMode, ModelWorkerBatch, ModelWorkerSamplingInfo
    rng = np.random.RandomState(seed)
    P = runner.page_size
    B = len(lens)
    ids = rng.randint(0, 1024, size=sum(lens)).astype(np.int32)
    pool = runner.req_to_token_pool
    locs = []
    nxt = P
    for b, n in enumerate(lens):
        slots = np.arange(nxt, nxt + n, dtype=np.int32)
        nxt += (n + P - 1) // P * P + P
        pool.write(b, 0, slots)
        locs.append(slots)
    rows, pos, pid = pool.take_page_deltas()
    return ModelWorkerBatch(
        bid=1, forward_mode=ForwardMode.EXTEND, input_ids=ids, req_pool_indices=np.arange(B, dtype=np.int32),
        seq_lens=np.asarray(lens, np.int32), out_cache_loc=np.concatenate(locs),
        positions=np.concatenate([np.arange(n, dtype=np.int32) for n in lens]),
        extend_prefix_lens=np.zeros(B, np.int32), extend_seq_lens=np.asarray(lens, np.int32),
        extend_logprob_start_lens=np.zeros(B, np.int32), page_delta_rows=rows, page_delta_pos=pos, page_delta_ids=pid,
        sampling_info=ModelWorkerSamplingInfo(np.ones(B, np.float32), np.ones(B, np.float32), np.ones(B, np.int32),
                                              np.zeros(B, np.float32), None, True, False, False, False))


def _decode_batch(runner, lens, tokens):
    from sglang_jax_b200.managers.schedule_batch import ForwardMode, ModelWorkerBatch, ModelWorkerSamplingInfo
    B = len(lens)
    pool = runner.req_to_token_pool
    locs = []
    for b, n in enumerate(lens):
        loc = int(pool.req_to_token[b, n - 1]) + 1
        pool.set_one(b, n, loc)
        locs.append(loc)
    rows, pos, pid = pool.take_page_deltas()
    return ModelWorkerBatch(
        bid=2, forward_mode=ForwardMode.DECODE, input_ids=np.asarray(tokens, np.int32),
        req_pool_indices=np.arange(B, dtype=np.int32), seq_lens=np.asarray(lens, np.int32) + 1,
        out_cache_loc=np.asarray(locs, np.int32), positions=np.asarray(lens, np.int32),
        page_delta_rows=rows, page_delta_pos=pos, page_delta_ids=pid,
        sampling_info=ModelWorkerSamplingInfo(np.ones(B, np.float32), np.ones(B, np.float32), np.ones(B, np.int32),
                                              np.zeros(B, np.float32), None, True, False, False, False))


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6)).item()


def test_forward_native_vs_reference(tiny_path):
    from sglang_jax_b200 import ops
    from sglang_jax_b200.ops import native
    runner, _ = _runner(tiny_path, disable_cuda_graph=True)
    lens = [5, 64, 130, 17]
    batch = _extend_batch(runner, lens)
    out_n, _, _ = runner.forward(batch, skip_sample=True)
    ops.set_force_reference(True)
    try:
        out_r, _, _ = runner.forward(batch, skip_sample=True)
    finally:
        ops.set_force_reference(False)
    torch.cuda.synchronize()
    native.check_status()
    assert _rel(out_n.next_token_logits, out_r.next_token_logits) < 3e-2
    toks = torch.argmax(out_r.next_token_logits, -1).tolist()
    dbatch = _decode_batch(runner, lens, toks)
    d_n, _, _ = runner.forward(dbatch, skip_sample=True)
    ops.set_force_reference(True)
    try:
        d_r, _, _ = runner.forward(dbatch, skip_sample=True)
    finally:
        ops.set_force_reference(False)
    torch.cuda.synchronize()
    native.check_status()
    assert _rel(d_n.next_token_logits, d_r.next_token_logits) < 3e-2


def test_cuda_graph_decode_matches_eager(tiny_path):
    from sglang_jax_b200.ops import native
    runner, _ = _runner(tiny_path, cuda_graph_max_bs=8)
    assert runner.cuda_graph_runner is not None and runner.cuda_graph_runner.graphs
    lens = [33, 64, 7]
    batch = _extend_batch(runner, lens, seed=3)
    out, ids, _ = runner.forward(batch)
    toks = ids.tolist()
    dbatch = _decode_batch(runner, lens, toks)
    assert runner.cuda_graph_runner.can_run(dbatch)
    _, g_ids, _ = runner.forward(dbatch)
    g_ids = g_ids.clone()
    runner.cuda_graph_runner.enabled = False
    _, e_ids, _ = runner.forward(dbatch)     # same slots, same inputs: idempotent
    torch.cuda.synchronize()
    native.check_status()
    assert g_ids.tolist() == e_ids.tolist()
    assert runner.graph_recaptures == 0 and runner.graph_replays == 1


def test_engine_generate_gpu(tiny_path):
    import os
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.ops import native
    from sglang_jax_b200.parallel import state as ps
    os.environ.pop("SGLB_GEMM_PLAN_LIBRARY", None)      # the engine's default: the plan may also pick the library GEMM
    ps.reset_state()
    outs = {}
    prompts = [list(range(1, 50)), list(range(3, 200)), [7] * 20]
    for mode in ("native", "reference"):
        ps.reset_state()
        eng = Engine(model_path=tiny_path, device="cuda", dtype="bfloat16", page_size=16, skip_tokenizer_init=True,
                     max_total_tokens=8192, max_running_requests=8, enable_single_process=True,
                     cuda_graph_max_bs=8, disable_custom_kernels=(mode == "reference"),
                     disable_cuda_graph=(mode == "reference"))
        try:
            o = eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 12, "temperature": 0.0,
                                                                 "ignore_eos": True})
            outs[mode] = [x["output_ids"] for x in o]
            info = eng.get_server_info()["internal_states"][0]
            assert info["cuda_graph_recaptures"] == 0
        finally:
            eng.shutdown()
    torch.cuda.synchronize()
    native.check_status()
    assert all(len(x) == 12 for x in outs["native"])
    # greedy paths agree on the first tokens (bf16 rounding may diverge late in a sequence)
    agree = sum(a[:4] == b[:4] for a, b in zip(outs["native"], outs["reference"]))
    assert agree >= 2, outs


def test_engine_mixed_chunk_and_penalties_gpu(tiny_path):
    """`--enable-mixed-chunk` on the GPU kernels: in a mixed step the prefill rows run on the extend kernel and the
    decode rows on the decode kernel; greedy output starts like the unmixed engine's.  A request with penalties
    (token counts kept on the device, outside the CUDA graphs) runs in the same engine."""
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.ops import native
    from sglang_jax_b200.parallel import state as ps
    prompts = [list(range(1, 50)), list(range(3, 200)), [7] * 20]
    sp = {"max_new_tokens": 12, "temperature": 0.0, "ignore_eos": True}
    outs = {}
    for mixed in (False, True):
        ps.reset_state()
        eng = Engine(model_path=tiny_path, device="cuda", dtype="bfloat16", page_size=16, skip_tokenizer_init=True,
                     max_total_tokens=8192, max_running_requests=8, enable_single_process=True, cuda_graph_max_bs=8,
                     enable_mixed_chunk=mixed, chunked_prefill_size=64)
        try:
            outs[mixed] = [x["output_ids"] for x in eng.generate(input_ids=prompts, sampling_params=sp)]
            if mixed:
                pen = eng.generate(input_ids=[7] * 20, sampling_params=dict(sp, frequency_penalty=1.5,
                                                                            presence_penalty=0.5, min_new_tokens=4))
                assert len(pen["output_ids"]) == 12
        finally:
            eng.shutdown()
    torch.cuda.synchronize()
    native.check_status()
    assert all(len(x) == 12 for x in outs[True])
    agree = sum(a[:4] == b[:4] for a, b in zip(outs[True], outs[False]))
    assert agree >= 2, outs


@pytest.mark.parametrize("algo,topk,steps,ndraft,page", [("STANDALONE", 1, 3, 4, 16), ("STANDALONE", 3, 3, 8, 16),
                                                         ("EAGLE", 2, 3, 6, 1)])
def test_speculative_decoding_gpu(tiny_path, algo, topk, steps, ndraft, page):
    """Draft + masked tree verification + KV compaction on the sm_100a kernels: sequences have the
    requested length, nothing leaks, and greedy output starts like the plain engine's."""
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.ops import native
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import TINY_QWEN3, write_tiny_eagle_checkpoint
    prompts = [list(range(1, 50)), list(range(3, 200)), [7] * 20]
    sp = {"max_new_tokens": 24, "temperature": 0.0, "ignore_eos": True}
    if algo == "EAGLE":
        cfg = dict(TINY_QWEN3, head_dim=128, num_attention_heads=8, num_key_value_heads=2, hidden_size=1024,
                   intermediate_size=2048, num_hidden_layers=3, torch_dtype="bfloat16", tie_word_embeddings=False)
        draft = write_tiny_eagle_checkpoint("/tmp/sglb200_test_eagle_gpu", cfg)
    else:
        draft = tiny_path
    common = dict(model_path=tiny_path, device="cuda", dtype="bfloat16", page_size=page, skip_tokenizer_init=True,
                  max_total_tokens=8192, max_running_requests=8, enable_single_process=True, cuda_graph_max_bs=8)
    ps.reset_state()
    eng = Engine(**common)
    try:
        ref_out = [x["output_ids"] for x in eng.generate(input_ids=prompts, sampling_params=sp)]
    finally:
        eng.shutdown()
    ps.reset_state()
    eng = Engine(**common, speculative_algorithm=algo, speculative_draft_model_path=draft,
                 speculative_num_steps=steps, speculative_eagle_topk=topk, speculative_num_draft_tokens=ndraft)
    try:
        outs = eng.generate(input_ids=prompts, sampling_params=sp)
        eng.scheduler.check_memory()
        sampled = eng.generate(input_ids=prompts[:2], sampling_params=dict(sp, temperature=0.7, top_p=0.9))
        eng.scheduler.check_memory()
    finally:
        eng.shutdown()
    torch.cuda.synchronize()
    native.check_status()
    got = [x["output_ids"] for x in outs]
    assert all(len(x) == 24 for x in got) and all(len(x["output_ids"]) == 24 for x in sampled)
    assert all(x["meta_info"]["spec_verify_ct"] > 0 for x in outs)
    agree = sum(a[:4] == b[:4] for a, b in zip(got, ref_out))
    assert agree >= 2, (got, ref_out)
    if algo == "STANDALONE":
        # the target drafting for itself is mostly accepted
        steps_used = sum(x["meta_info"]["spec_verify_ct"] for x in outs)
        assert steps_used < 24 * len(prompts) * 0.8, steps_used


def test_deepseek_mla_decode_kernel_in_model(tmp_path):
    """A DeepSeek-shaped model (latent 512 + 64 rotary lanes, MoE) on the GPU: decode with the MLA
    kernel (eager and under the CUDA graph) against the same step through the PyTorch statements."""
    import json
    from sglang_jax_b200 import ops
    from sglang_jax_b200.ops import native
    cfg = dict(architectures=["DeepseekV3ForCausalLM"], model_type="deepseek_v3", hidden_size=512,
               intermediate_size=1024, moe_intermediate_size=256, num_hidden_layers=2, num_attention_heads=16,
               num_key_value_heads=16, q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
               v_head_dim=128, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2, n_group=1, topk_group=1,
               scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True, routed_scaling_factor=2.5,
               first_k_dense_replace=1, moe_layer_freq=1, rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=1024,
               tie_word_embeddings=False, max_position_embeddings=4096, torch_dtype="bfloat16")
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    lens = [5, 64, 130, 700]
    runner, _ = _runner(str(tmp_path), load_format="dummy", cuda_graph_max_bs=8)
    assert runner.cuda_graph_runner is not None and runner.cuda_graph_runner.graphs
    batch = _extend_batch(runner, lens)
    out, ids, _ = runner.forward(batch)
    toks = ids.tolist()
    dbatch = _decode_batch(runner, lens, toks)
    assert runner.cuda_graph_runner.can_run(dbatch)
    _, g_ids, _ = runner.forward(dbatch)                       # replayed graph with the MLA kernel inside
    g_ids = g_ids.clone()
    runner.cuda_graph_runner.enabled = False
    calls = {"n": 0}
    orig = native.mla_decode

    def counted(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)

    native.mla_decode = counted
    try:
        d_n, e_ids, _ = runner.forward(dbatch, skip_sample=False)
        d_n, _, _ = runner.forward(dbatch, skip_sample=True)
        assert calls["n"] == 4                                 # one launch per layer and forward
    finally:
        native.mla_decode = orig
    ops.set_force_reference(True)
    try:
        d_r, _, _ = runner.forward(dbatch, skip_sample=True)
    finally:
        ops.set_force_reference(False)
    torch.cuda.synchronize()
    native.check_status()
    assert g_ids.tolist() == e_ids.tolist()
    assert _rel(d_n.next_token_logits, d_r.next_token_logits) < 4e-2


def test_qwen3_moe_fp8_recipe_runs_on_grouped_fp8_gemm(tmp_path):
    """A Qwen3-MoE-shaped model under the dynamic fp8 recipe: experts keep fp8 storage, every MoE layer runs
    the grouped fp8 GEMM path (prefill eager, decode inside the CUDA graph) and one expert layer in isolation
    agrees with the PyTorch statement of the same quantised experts."""
    import json
    from sglang_jax_b200 import ops
    from sglang_jax_b200.layers.moe import FusedMoE
    from sglang_jax_b200.ops import moe_native, native
    cfg = dict(architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", hidden_size=512, intermediate_size=1024,
               moe_intermediate_size=256, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
               head_dim=128, num_experts=16, num_experts_per_tok=4, norm_topk_prob=True, decoder_sparse_step=1,
               mlp_only_layers=[], rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=1024, tie_word_embeddings=False,
               max_position_embeddings=4096, torch_dtype="bfloat16")
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    runner, _ = _runner(str(tmp_path), load_format="dummy", cuda_graph_max_bs=8, quantization="fp8_qwen3_30b_a3b")
    moes = [m for m in runner.model.modules() if isinstance(m, FusedMoE)]
    assert len(moes) == 2 and all(m.fp8 and m.w13_weight.dtype == torch.float8_e4m3fn for m in moes)
    calls = {"n": 0}
    orig = moe_native.fused_experts_fp8

    def counted(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)

    moe_native.fused_experts_fp8 = counted
    lens = [5, 64, 130, 300]
    try:
        batch = _extend_batch(runner, lens)
        out, ids, _ = runner.forward(batch)
        assert calls["n"] == 2
        dbatch = _decode_batch(runner, lens, ids.tolist())
        assert runner.cuda_graph_runner.can_run(dbatch)
        _, g_ids, _ = runner.forward(dbatch)
        g_ids = g_ids.clone()
        runner.cuda_graph_runner.enabled = False
        e_out, e_ids, _ = runner.forward(dbatch)
        assert calls["n"] == 4
    finally:
        moe_native.fused_experts_fp8 = orig
    torch.cuda.synchronize()
    native.check_status()
    assert torch.isfinite(out.next_token_logits).all() and out.next_token_logits.float().std() > 1e-3
    # The graph sizes the split-KV decode attention for the longest context it may meet, the eager step for the
    # lengths at hand: the summation order differs, so a token may differ only where the two best logits tie.
    lg = e_out.next_token_logits.float()
    for i, (g, e) in enumerate(zip(g_ids.tolist(), e_ids.tolist())):
        if g != e:
            assert float(lg[i].max() - lg[i, g]) < 0.1 * float(lg[i].std()), (i, g, e, float(lg[i].max() - lg[i, g]))
    assert sum(g == e for g, e in zip(g_ids.tolist(), e_ids.tolist())) >= 3
    moe = moes[0]
    x = (torch.randn(77, 512, device="cuda") * 0.5).bfloat16()
    tw, tid = ops.topk_route(torch.randn(77, 16, device="cuda"), 4)
    y_n = moe(x, tw, tid)
    ops.set_force_reference(True)
    try:
        y_r = moe(x, tw, tid)
    finally:
        ops.set_force_reference(False)
    assert y_r.float().std() > 0 and _rel(y_n, y_r) < 2e-2


def test_qwen3_next_decode_with_recurrent_kernels(tmp_path):
    """Hybrid Gated-DeltaNet model on the GPU: a decode step through the in-place recurrent kernels
    equals the same step through the PyTorch statements, including the updated state pools."""
    import json
    from sglang_jax_b200 import ops
    from sglang_jax_b200.ops import native
    cfg = dict(architectures=["Qwen3NextForCausalLM"], model_type="qwen3_next", hidden_size=512, intermediate_size=1024,
               num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6,
               vocab_size=1024, max_position_embeddings=4096, full_attention_interval=2, linear_num_key_heads=2,
               linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=128, linear_conv_kernel_dim=4,
               partial_rotary_factor=0.25, num_experts=0, tie_word_embeddings=False, torch_dtype="bfloat16",
               layer_types=["linear_attention", "full_attention"] * 2)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    runner, _ = _runner(str(tmp_path), load_format="dummy", disable_cuda_graph=True, disable_radix_cache=True)
    lens = [5, 64, 130]
    out, ids, _ = runner.forward(_extend_batch(runner, lens))
    toks = ids.tolist()
    pool = runner.recurrent_pool
    conv0, rec0 = pool.conv_state.clone(), pool.recurrent_state.clone()
    calls = {"n": 0}
    orig = native.delta_rule_step

    def counted(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)

    native.delta_rule_step = counted
    try:
        dbatch = _decode_batch(runner, lens, toks)
        d_n, _, _ = runner.forward(dbatch, skip_sample=True)
    finally:
        native.delta_rule_step = orig
    assert calls["n"] == 2                                     # the two linear-attention layers
    conv_n, rec_n = pool.conv_state.clone(), pool.recurrent_state.clone()
    pool.conv_state.copy_(conv0)
    pool.recurrent_state.copy_(rec0)
    ops.set_force_reference(True)
    try:
        d_r, _, _ = runner.forward(dbatch, skip_sample=True)
    finally:
        ops.set_force_reference(False)
    torch.cuda.synchronize()
    native.check_status()
    assert _rel(d_n.next_token_logits, d_r.next_token_logits) < 4e-2
    assert _rel(rec_n, pool.recurrent_state) < 2e-2 and _rel(conv_n, pool.conv_state) < 2e-2


_QWEN3_NEXT_TINY = dict(
    architectures=["Qwen3NextForCausalLM"], model_type="qwen3_next", hidden_size=512, intermediate_size=1024,
    num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6,
    vocab_size=1024, max_position_embeddings=4096, full_attention_interval=2, linear_num_key_heads=2,
    linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=128, linear_conv_kernel_dim=4,
    partial_rotary_factor=0.25, num_experts=0, tie_word_embeddings=False, torch_dtype="bfloat16",
    layer_types=["linear_attention", "full_attention"] * 2)
_GEMMA2_TINY = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2", hidden_size=512, intermediate_size=1024,
    num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6,
    rope_theta=10000.0, vocab_size=1024, tie_word_embeddings=True, max_position_embeddings=4096, sliding_window=48,
    query_pre_attn_scalar=128, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
    hidden_activation="gelu_pytorch_tanh", torch_dtype="bfloat16")


@pytest.mark.parametrize("name,cfg,extra", [("qwen3_next", _QWEN3_NEXT_TINY, dict(disable_radix_cache=True)),
                                            ("gemma2", _GEMMA2_TINY, dict())])
def test_hybrid_models_decode_inside_cuda_graphs(tmp_path, name, cfg, extra):
    """Hybrid linear-attention (recurrent state pool) and hybrid sliding-window (dual KV pool) models decode
    through captured CUDA graphs: the graphs are replayed, nothing is recaptured and greedy output equals the
    eager engine's, including sequences that run past the window."""
    import json
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.ops import native
    from sglang_jax_b200.parallel import state as ps
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    prompts = [list(range(1, 40)), list(range(3, 150)), [7, 9, 11] * 9]
    outs = {}
    for graphs in (True, False):
        ps.reset_state()
        eng = Engine(model_path=str(tmp_path), device="cuda", dtype="bfloat16", page_size=16, skip_tokenizer_init=True,
                     max_total_tokens=8192, max_running_requests=8, enable_single_process=True, load_format="dummy",
                     cuda_graph_max_bs=8, disable_cuda_graph=not graphs, disable_overlap_schedule=True, **extra)
        try:
            o = eng.generate(input_ids=prompts, sampling_params={"max_new_tokens": 24, "temperature": 0.0,
                                                                 "ignore_eos": True})
            outs[graphs] = [x["output_ids"] for x in o]
            info = eng.get_server_info()["internal_states"][0]
            assert info["cuda_graph_recaptures"] == 0
            assert (info["cuda_graph_replays"] >= 20) if graphs else (info["cuda_graph_replays"] == 0)
        finally:
            eng.shutdown()
    torch.cuda.synchronize()
    native.check_status()
    assert all(len(x) == 24 for x in outs[True])
    assert len({t for o in outs[True] for t in o}) > 3
    # the captured step sizes its attention splits for the longest context, so late tokens may round differently
    assert all(a[:8] == b[:8] for a, b in zip(outs[True], outs[False])), outs
    assert sum(a == b for a, b in zip(outs[True], outs[False])) >= 2, outs


def test_sampled_decode_runs_inside_cuda_graphs(tiny_path):
    """Temperature / top-k / top-p requests without their own seed decode through the sampled graph variant
    (sampling kernel inside the graph): graphs are replayed, nothing is recaptured, two engines with the same
    seed agree token for token, equal prompts in one batch draw different continuations, and every token lies in
    the top-k set of an eager forward of its prefix."""
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.ops import native
    from sglang_jax_b200.parallel import state as ps
    prompts = [list(range(1, 50)), list(range(1, 50)), [7, 9, 11] * 9, list(range(3, 120))]
    sp = {"max_new_tokens": 16, "temperature": 1.5, "top_k": 8, "top_p": 0.95, "ignore_eos": True}
    runs = []
    for _ in range(2):
        ps.reset_state()
        eng = Engine(model_path=tiny_path, device="cuda", dtype="bfloat16", page_size=16, skip_tokenizer_init=True,
                     max_total_tokens=8192, max_running_requests=8, enable_single_process=True, cuda_graph_max_bs=8,
                     random_seed=11)
        try:
            o = eng.generate(input_ids=prompts, sampling_params=sp)
            runs.append([x["output_ids"] for x in o])
            info = eng.get_server_info()["internal_states"][0]
            assert info["cuda_graph_recaptures"] == 0 and info["cuda_graph_replays"] >= 14
            greedy = eng.generate(input_ids=prompts[:1], sampling_params={"max_new_tokens": 16, "temperature": 0.0,
                                                                          "ignore_eos": True})[0]["output_ids"]
        finally:
            eng.shutdown()
    torch.cuda.synchronize()
    native.check_status()
    assert runs[0] == runs[1]
    assert all(len(x) == 16 for x in runs[0])
    assert runs[0][0] != runs[0][1]                          # same prompt, different per-row seeds
    assert runs[0][0] != greedy and runs[0][1] != greedy
    # the last drawn token lies in the top-k set of an eager forward of everything before it (a few ranks of
    # slack for bf16 rounding between the chunked prefill here and the decode steps there)
    runner, _ = _runner(tiny_path, disable_cuda_graph=True)
    for p, o in zip(prompts[2:], runs[0][2:]):
        seq = p + o[:-1]
        batch = _extend_batch(runner, [len(seq)])
        batch.input_ids = np.asarray(seq, np.int32)
        out, _, _ = runner.forward(batch, skip_sample=True)
        assert o[-1] in out.next_token_logits[-1].float().topk(12).indices.tolist()


def test_fp8_recipe_runs_on_the_fp8_gemm(tiny_path):
    """`--quantization fp8` (per-channel e4m3 weights, per-token e4m3 activations): the projections go
    through the fp8 tensor-core GEMM and agree with the same quantised model evaluated in PyTorch."""
    from sglang_jax_b200 import ops
    from sglang_jax_b200.ops import native
    runner, _ = _runner(tiny_path, disable_cuda_graph=True, quantization="fp8")
    calls = {"n": 0}
    orig = native.gemm_fp8

    def counted(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)

    native.gemm_fp8 = counted
    try:
        batch = _extend_batch(runner, [5, 64, 130, 17])
        out_n, _, _ = runner.forward(batch, skip_sample=True)
    finally:
        native.gemm_fp8 = orig
    assert calls["n"] == 3 * 4                                  # qkv, o, gate_up, down in each of the three layers
    ops.set_force_reference(True)
    try:
        out_r, _, _ = runner.forward(batch, skip_sample=True)
    finally:
        ops.set_force_reference(False)
    torch.cuda.synchronize()
    native.check_status()
    # end to end the two paths round differently (bf16 de-quantised operands vs exact fp8 products, and
    # every later activation is re-quantised), so only a loose bound holds on random weights
    assert _rel(out_n.next_token_logits, out_r.next_token_logits) < 0.2
    # one projection in isolation is tight
    lin = runner.model.model.layers[0].mlp.gate_up_proj
    x = (torch.randn(37, lin.qweight.qweight.shape[1], device="cuda") * 0.5).bfloat16()
    y_n = lin(x)
    ops.set_force_reference(True)
    try:
        y_r = lin(x)
    finally:
        ops.set_force_reference(False)
    assert _rel(y_n, y_r) < 2e-2


def test_qwen2_5_vl_vision_tower_uses_varlen_attention_on_gpu():
    """The vision tower on the GPU (windowed and full-attention blocks as packed segments through the varlen
    kernel, head dim 80 padded to 128) agrees with the same weights through the PyTorch path."""
    from types import SimpleNamespace
    from sglang_jax_b200 import ops
    from sglang_jax_b200.multimodal.models.qwen2_5_vl_vit import Qwen2_5_VisionTransformer
    from sglang_jax_b200.ops import native
    cfg = SimpleNamespace(depth=4, hidden_size=320, intermediate_size=512, num_heads=4, in_channels=3, patch_size=14,
                          spatial_merge_size=2, temporal_patch_size=2, window_size=112, fullatt_block_indexes=[1, 3],
                          out_hidden_size=256, hidden_act="silu")
    torch.manual_seed(0)
    vit = Qwen2_5_VisionTransformer(cfg, dtype=torch.bfloat16).cuda()
    for p in vit.parameters():
        p.data.normal_(0, 0.05) if p.dim() > 1 else p.data.uniform_(0.5, 1.5)
    grid = torch.tensor([[1, 12, 20], [1, 8, 8], [2, 4, 6]])
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(n, 3 * 2 * 14 * 14, device="cuda").bfloat16()
    calls = {"n": 0}
    orig = native.varlen_attention

    def counted(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)

    native.varlen_attention = counted
    try:
        got = vit(px, grid)
    finally:
        native.varlen_attention = orig
    assert calls["n"] == 4
    ops.set_force_reference(True)
    try:
        want = vit(px, grid)
    finally:
        ops.set_force_reference(False)
    torch.cuda.synchronize()
    native.check_status()
    assert got.shape == want.shape == (n // 4, 256) and want.float().std() > 1e-3
    assert _rel(got, want) < 3e-2


def test_encoders_use_varlen_attention_on_gpu():
    """Qwen3-Omni vision and audio encoders and the Kimi-K2.5 vision tower on the GPU: frames / windows / items as
    packed segments through the varlen kernel (head dims 72, 64, 72) agree with the PyTorch path of the same weights."""
    from types import SimpleNamespace
    from sglang_jax_b200 import ops
    from sglang_jax_b200.multimodal.model_executor.loading import init_dummy
    from sglang_jax_b200.multimodal.models.kimi_k25.kimi_k25_vit import KimiK25VisionModel
    from sglang_jax_b200.multimodal.models.qwen3_omni.audio_encoder import Qwen3OmniMoeAudioEncoder
    from sglang_jax_b200.multimodal.models.qwen3_omni.vision_encoder import Qwen3OmniMoeVisionEncoder
    from sglang_jax_b200.ops import native
    bf = torch.bfloat16
    g = torch.Generator().manual_seed(0)
    vcfg = SimpleNamespace(depth=3, hidden_size=288, intermediate_size=384, num_heads=4, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=128, num_position_embeddings=144,
                           deepstack_visual_indexes=[0, 2], hidden_act="gelu_pytorch_tanh")
    vis = init_dummy(Qwen3OmniMoeVisionEncoder(vcfg, dtype=bf), seed=1, std=0.05).cuda().eval()
    grid = torch.tensor([[1, 12, 20], [2, 8, 8]])
    px = torch.randn(int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * 4 * 4, generator=g).cuda().to(bf)
    acfg = SimpleNamespace(num_mel_bins=16, d_model=256, encoder_layers=2, encoder_attention_heads=4,
                           encoder_ffn_dim=512, downsample_hidden_size=8, output_dim=64, max_source_positions=64,
                           n_window=50, n_window_infer=200, conv_chunksize=4, activation_function="gelu",
                           scale_embedding=False)
    aud = init_dummy(Qwen3OmniMoeAudioEncoder(acfg, dtype=bf), seed=2, std=0.05).cuda().eval()
    feats, flens = torch.randn(16, 157 + 330, generator=g).cuda().to(bf), torch.tensor([157, 330])
    kcfg = SimpleNamespace(patch_size=4, in_channels=3, vt_hidden_size=288, vt_num_attention_heads=4,
                           vt_intermediate_size=384, vt_num_hidden_layers=2, init_pos_emb_height=6, init_pos_emb_width=6,
                           init_pos_emb_time=4, merge_kernel_size=[2, 2], text_hidden_size=64)
    kimi = init_dummy(KimiK25VisionModel(kcfg, dtype=bf), seed=3, std=0.05).cuda().eval()
    kpx = torch.randn(36 + 64, 3, 4, 4, generator=g).cuda().to(bf)
    runs = [lambda: vis(px, grid), lambda: aud(feats, flens), lambda: kimi(kpx, [[1, 6, 6], [2, 4, 8]])]
    calls = {"n": 0}
    orig = native.varlen_attention

    def counted(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)

    for run, layers in zip(runs, (3, 2, 2)):
        calls["n"] = 0
        native.varlen_attention = counted
        try:
            with torch.inference_mode():
                got = run()
        finally:
            native.varlen_attention = orig
        assert calls["n"] == layers
        ops.set_force_reference(True)
        try:
            with torch.inference_mode():
                want = run()
        finally:
            ops.set_force_reference(False)
        torch.cuda.synchronize()
        native.check_status()
        assert got.shape == want.shape and want.float().std() > 1e-3
        assert _rel(got, want) < 4e-2


def test_wan_dit_self_attention_uses_the_varlen_kernel_on_gpu():
    """The diffusion transformer's dense bidirectional self-attention runs on the varlen attention kernel (head dim
    128: tcgen05); the block's output follows the PyTorch SDPA path."""
    from types import SimpleNamespace
    from sglang_jax_b200 import ops
    from sglang_jax_b200.multimodal.models.dit import WanTransformer3DModel
    from sglang_jax_b200.ops import native
    cfg = SimpleNamespace(in_channels=4, out_channels=4, patch_size=(1, 2, 2), num_attention_heads=4,
                          attention_head_dim=128, ffn_dim=1024, num_layers=2, text_dim=64, freq_dim=64)
    torch.manual_seed(0)
    m = WanTransformer3DModel(cfg, dtype=torch.bfloat16).cuda()
    for p in m.parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.03)
    lat = torch.randn(2, 4, 3, 16, 16, device="cuda").bfloat16()       # 2 x (3 * 8 * 8 = 192 tokens)
    t = torch.tensor([500.0, 20.0], device="cuda")
    text = torch.randn(2, 7, 64, device="cuda").bfloat16()
    calls = {"n": 0}
    orig = native.varlen_attention

    def counted(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)

    native.varlen_attention = counted
    try:
        got = m(lat, t, text)
    finally:
        native.varlen_attention = orig
    assert calls["n"] == 2                                              # one per block
    ops.set_force_reference(True)
    try:
        want = m(lat, t, text)
    finally:
        ops.set_force_reference(False)
    torch.cuda.synchronize()
    native.check_status()
    assert torch.isfinite(got).all()
    err = (got.float() - want.float()).abs().max().item()
    assert err < 0.05 * want.float().abs().max().item() + 0.02, err
