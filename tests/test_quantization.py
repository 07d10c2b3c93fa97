"""Quantisation helpers, presets, static-FP8 checkpoint ingestion and a quantised engine run
(reference tests: `python/sgl_jax/test/quantization/`)."""

import json
import os

import pytest
import torch

from sglang_jax_b200.configs.quantization_config import QuantizationConfig, presets
from sglang_jax_b200.model_loader.loader import dequant_static_fp8
from sglang_jax_b200.utils.quantization import (dequantize_tensor, quantize_activation, quantize_tensor)


@pytest.mark.parametrize("dtype,tol", [(torch.float8_e4m3fn, 0.07), (torch.int8, 0.02)])
@pytest.mark.parametrize("gran,bs", [("per_tensor", None), ("per_channel", None), ("block", (128, 128)), ("block", (64, 32))])
def test_quantize_roundtrip(dtype, tol, gran, bs):
    g = torch.Generator().manual_seed(0)
    w = torch.randn(200, 300, generator=g) * torch.linspace(0.1, 3.0, 200).view(-1, 1)
    q, s = quantize_tensor(w, dtype, gran, bs)
    assert q.dtype == dtype and q.shape == w.shape
    if gran == "block":
        assert s.shape == (-(-200 // bs[0]), -(-300 // bs[1]))
    back = dequantize_tensor(q, s, bs, torch.float32)
    rel = (back - w).abs().max() / w.abs().max()
    assert rel < tol, rel
    if gran != "per_tensor":
        # finer scales never do worse than one scale for the whole tensor
        q0, s0 = quantize_tensor(w, dtype, "per_tensor")
        assert (back - w).pow(2).mean() <= (dequantize_tensor(q0, s0, None, torch.float32) - w).pow(2).mean() * 1.01


def test_activation_group_scales():
    x = torch.randn(7, 300)
    q, s = quantize_activation(x, torch.float8_e4m3fn, 128)
    assert s.shape == (7, 3)
    back = q.float() * s.repeat_interleave(128, 1)[:, :300]
    assert (back - x).abs().max() / x.abs().max() < 0.07


def test_presets_parse_and_rules():
    names = presets()
    assert {"fp8", "fp8_deepseek_v3", "int8", "fp8_block_128_dynamic", "int8_w8a8"} <= set(names)
    for n in names:
        cfg = QuantizationConfig.resolve(n)
        assert cfg.linear_rules, n
    ds = QuantizationConfig.resolve("fp8_deepseek_v3")
    assert ds.is_static_checkpoint and ds.weight_block_size == (128, 128) and ds.granularity == "block"
    q = QuantizationConfig.resolve("fp8_qwen3_30b_a3b")
    assert q.rule_for("model.layers.0.mlp.gate") is None
    assert q.rule_for("model.layers.0.self_attn.qkv_proj").weight_dtype == torch.float8_e4m3fn

    class HF:
        quantization_config = {"quant_method": "fp8", "weight_block_size": [128, 128]}
    assert QuantizationConfig.resolve(None, None, HF()).is_static_checkpoint
    with pytest.raises(ValueError):
        QuantizationConfig.resolve("nope")


def test_static_fp8_stream_is_folded_in_any_order():
    w = torch.randn(256, 384)
    q, s = quantize_tensor(w, torch.float8_e4m3fn, "block", (128, 128))
    want = dequantize_tensor(q, s, (128, 128), torch.float32)
    plain = torch.randn(4, 4)
    for order in ([("a.weight", q), ("a.weight_scale_inv", s), ("b.weight", plain)],
                  [("a.weight_scale_inv", s), ("b.weight", plain), ("a.weight", q)]):
        out = dict(dequant_static_fp8(iter(order)))
        assert set(out) == {"a.weight", "b.weight"}
        assert out["a.weight"].dtype == torch.float32 and torch.equal(out["a.weight"], want)
        assert torch.equal(out["b.weight"], plain)


def test_engine_runs_static_fp8_checkpoint_and_dynamic_recipes(tmp_path):
    """A block-FP8 copy of the tiny checkpoint is served in its own format (weights back on the checkpoint's block
    grid, per-token-group-128 fp8 activations): it must reproduce the run of the 128 x 128 dynamic recipe over its
    de-quantised weights exactly; dynamic recipes must run."""
    from safetensors.torch import save_file
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.utils.tiny_models import TINY_QWEN3, tiny_qwen3_state_dict, write_config_only
    sd = tiny_qwen3_state_dict(TINY_QWEN3, 0)
    fp8_sd, deq_sd = {}, {}
    for k, v in sd.items():
        if v.dim() == 2 and "embed" not in k:
            q, s = quantize_tensor(v, torch.float8_e4m3fn, "block", (128, 128))
            fp8_sd[k] = q
            fp8_sd[k + "_scale_inv"] = s
            deq_sd[k] = dequantize_tensor(q, s, (128, 128), torch.float32)
        else:
            fp8_sd[k] = v
            deq_sd[k] = v
    paths = {}
    for name, d, extra in (("fp8", fp8_sd, {"quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}}),
                           ("deq", deq_sd, {}), ("dense", sd, {})):
        p = write_config_only(str(tmp_path / name), dict(TINY_QWEN3, **extra))
        save_file({k: v.contiguous() for k, v in d.items()}, os.path.join(p, "model.safetensors"))
        paths[name] = p
    prompts = [[3, 17, 42, 9, 5, 11, 8], [4, 4, 19, 23]]
    sp = {"temperature": 0.0, "max_new_tokens": 8, "ignore_eos": True}

    def run(path, **kw):
        ps.reset_state()
        eng = Engine(model_path=path, device="cpu", enable_single_process=True, page_size=4, skip_tokenizer_init=True,
                     max_total_tokens=1024, dtype="float32", log_level="error", **kw)
        try:
            return [o["output_ids"] for o in eng.generate(input_ids=prompts, sampling_params=sp)]
        finally:
            eng.shutdown()

    a, b = run(paths["fp8"]), run(paths["deq"], quantization="fp8_block_128_dynamic")
    assert a == b
    dense = run(paths["dense"])
    for recipe in ("fp8", "int8", "fp8_block_128_dynamic"):
        got = run(paths["dense"], quantization=recipe)
        assert all(len(g) == 8 for g in got), recipe
    del dense


def test_quantized_linear_is_close_to_dense():
    from sglang_jax_b200.utils.quantization import QuantizedWeight
    g = torch.Generator().manual_seed(1)
    w = torch.randn(96, 256, generator=g)
    x = torch.randn(5, 256, generator=g)
    want = x @ w.t()
    for dtype, gran, bs, act in ((torch.float8_e4m3fn, "per_channel", None, torch.float8_e4m3fn),
                                 (torch.int8, "per_channel", None, torch.int8),
                                 (torch.float8_e4m3fn, "block", (128, 128), torch.float8_e4m3fn),
                                 (torch.float8_e4m3fn, "block", (128, 128), None)):
        q, s = quantize_tensor(w, dtype, gran, bs)
        y = QuantizedWeight(q, s, bs, act, torch.float32).linear(x)
        rel = (y - want).norm() / want.norm()
        assert rel < 0.06, (dtype, gran, rel)


def test_fused_moe_fp8_storage_keeps_only_quantised_experts():
    """A W8A8 e4m3 per-channel recipe replaces the expert tensors with fp8 storage + fp32 scales and the
    forward stays close to the unquantised experts; block recipes keep de-quantised compute-dtype storage."""
    from sglang_jax_b200.layers.moe import FusedMoE
    from sglang_jax_b200.ops import reference
    torch.manual_seed(0)
    moe = FusedMoE(4, 64, 32, tp_size=1, tp_rank=0, ep_size=1)
    moe.w13_weight.data.normal_(0, 0.1)
    moe.w2_weight.data.normal_(0, 0.1)
    x = torch.randn(12, 64).bfloat16()
    ids = torch.stack([torch.randperm(4)[:2] for _ in range(12)]).int()
    w = torch.rand(12, 2)
    add = torch.randn(12, 64).bfloat16()
    want = reference.moe_forward(x, moe.w13_weight, moe.w2_weight, w, ids, 0).float() + add.float()
    blocky = FusedMoE(4, 64, 32, tp_size=1, tp_rank=0, ep_size=1)
    blocky.load_state_dict(moe.state_dict())
    blocky.quantize_(torch.float8_e4m3fn, (16, 16), torch.float8_e4m3fn)
    assert not blocky.fp8 and blocky.w13_weight.dtype == torch.bfloat16
    moe.quantize_(torch.float8_e4m3fn, None, torch.float8_e4m3fn)
    assert moe.fp8 and moe.w13_weight.dtype == torch.float8_e4m3fn and moe.w2_weight.dtype == torch.float8_e4m3fn
    assert sorted(n for n, _ in moe.named_parameters()) == ["w13_weight", "w2_weight"]
    assert sorted(n for n, _ in moe.named_buffers()) == ["w13_scale", "w2_scale"]
    assert moe.w13_scale.shape == (4, 64) and moe.w2_scale.shape == (4, 64)
    got = moe(x, w, ids, add=add).float()
    assert got.std() > 0.05
    assert ((got - want).norm() / want.norm()).item() < 0.08
    w13, w2 = moe._bf16_weights()
    assert w13.shape == (4, 64, 64) and w2.dtype == torch.bfloat16


def test_experts_built_in_fp8_storage_quantise_while_loading():
    """Under `expert_storage(e4m3)` the experts never exist in bf16: per-expert checkpoint tensors are quantised by
    the weight loader, and the result equals quantising a bf16-loaded layer afterwards (tensor-parallel slices too)."""
    from sglang_jax_b200.layers.moe import FusedMoE, expert_storage
    torch.manual_seed(0)
    E, H, I = 4, 64, 64
    gate = [torch.randn(I, H).bfloat16() * 0.1 for _ in range(E)]
    up = [torch.randn(I, H).bfloat16() * 0.1 for _ in range(E)]
    down = [torch.randn(H, I).bfloat16() * 0.1 for _ in range(E)]
    for tp, rank in ((1, 0), (2, 1)):
        plain = FusedMoE(E, H, I, tp_size=tp, tp_rank=rank, ep_size=1)
        with expert_storage(torch.float8_e4m3fn):
            lean = FusedMoE(E, H, I, tp_size=tp, tp_rank=rank, ep_size=1)
        assert lean.fp8 and lean.w13_weight.dtype == torch.float8_e4m3fn and not plain.fp8
        for m in (plain, lean):
            for e in range(E):
                m.weight_loader(m.w13_weight, gate[e], "gate", e)
                m.weight_loader(m.w13_weight, up[e], "up", e)
                m.weight_loader(m.w2_weight, down[e], "down", e)
        plain.quantize_(torch.float8_e4m3fn, None, torch.float8_e4m3fn)
        assert plain.fp8
        assert torch.equal(plain.w13_weight.view(torch.uint8), lean.w13_weight.view(torch.uint8))
        assert torch.equal(plain.w2_weight.view(torch.uint8), lean.w2_weight.view(torch.uint8))
        assert torch.equal(plain.w13_scale, lean.w13_scale) and torch.equal(plain.w2_scale, lean.w2_scale)
        lean.quantize_(torch.float8_e4m3fn, None, torch.float8_e4m3fn)             # a no-op on fp8-built experts
        x = torch.randn(9, H).bfloat16()
        ids = torch.stack([torch.randperm(E)[:2] for _ in range(9)]).int()
        w = torch.rand(9, 2)
        assert torch.equal(lean(x, w, ids), plain(x, w, ids))
    # float32 experts (CPU reference runs) keep the compute-dtype storage
    with expert_storage(torch.float8_e4m3fn):
        assert not FusedMoE(E, H, I, dtype=torch.float32, tp_size=1, tp_rank=0, ep_size=1).fp8


def test_dummy_loader_builds_fp8_experts_for_w8a8_recipes(tmp_path):
    import json
    from sglang_jax_b200.configs.model_config import ModelConfig
    from sglang_jax_b200.configs.quantization_config import QuantizationConfig
    from sglang_jax_b200.layers.moe import FusedMoE
    from sglang_jax_b200.model_loader.loader import DummyModelLoader
    from sglang_jax_b200.parallel import state as ps
    from sglang_jax_b200.server_args import ServerArgs
    cfg = dict(architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", hidden_size=64, intermediate_size=128,
               moe_intermediate_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
               num_experts=4, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[],
               rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=128, tie_word_embeddings=False,
               max_position_embeddings=256, torch_dtype="bfloat16")
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    ps.reset_state()
    ps.init_distributed(0, 1, "cpu")
    sa = ServerArgs(model_path=str(tmp_path), device="cpu", dtype="bfloat16", skip_tokenizer_init=True,
                    load_format="dummy", quantization="fp8_qwen3_30b_a3b")
    mc = ModelConfig.from_server_args(sa)
    model = DummyModelLoader(0).load_model(mc, "cpu", QuantizationConfig.resolve("fp8_qwen3_30b_a3b"))
    moes = [m for m in model.modules() if isinstance(m, FusedMoE)]
    assert len(moes) == 2 and all(m.fp8 and m.w13_weight.dtype == torch.float8_e4m3fn for m in moes)
    eff = moes[0]._bf16_weights()[0].float()
    assert 0.01 < eff.std().item() < 0.04                     # e4m3 normal(0, 1) values times the 0.02 default scale
