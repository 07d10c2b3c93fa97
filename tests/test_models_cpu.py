"""Model families against HF transformers in fp32 on CPU (greedy tokens must match exactly)."""

import json
import os

import pytest
import torch
from safetensors.torch import save_file


def _save(path, hf_model, cfg: dict, arch: str, model_type: str, rename=None):
    os.makedirs(path, exist_ok=True)
    sd = {k: v.contiguous().clone() for k, v in hf_model.state_dict().items()}
    if cfg.get("tie_word_embeddings"):
        sd.pop("lm_head.weight", None)
    if rename:
        sd = rename(sd)
    save_file(sd, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(dict(cfg, architectures=[arch], model_type=model_type, torch_dtype="float32"), f)
    return path


def _generate(path, ids, n=10, **kw):
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    ps.reset_state()
    eng = Engine(model_path=path, device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                 max_total_tokens=4096, enable_single_process=True, **kw)
    try:
        outs = eng.generate(input_ids=ids, sampling_params={"max_new_tokens": n, "temperature": 0, "ignore_eos": True})
        return [o["output_ids"] for o in outs]
    finally:
        eng.shutdown()


def _hf_generate(hf, ids, n=10):
    out = []
    for i in ids:
        with torch.no_grad():
            out.append(hf.generate(torch.tensor([i]), max_new_tokens=n, do_sample=False)[0, len(i):].tolist())
    return out


PROMPTS = [list(range(5, 40)), [9, 8, 7, 6, 5, 4, 3] * 5, [100, 200, 300]]


def _init(hf, std=0.05):
    torch.manual_seed(0)
    for p in hf.parameters():
        if p.dim() > 1:
            p.data.normal_(0, std)
    return hf.float().eval()


def test_llama_matches_hf(tmp_path):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, rms_norm_eps=1e-5, rope_theta=500000.0, vocab_size=512,
               tie_word_embeddings=False, max_position_embeddings=512,
               rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 64})
    hf = _init(LlamaForCausalLM(LlamaConfig(**cfg)))
    path = _save(str(tmp_path / "llama"), hf, cfg, "LlamaForCausalLM", "llama")
    assert _generate(path, PROMPTS) == _hf_generate(hf, PROMPTS)


def test_qwen2_bias_matches_hf(tmp_path):
    from transformers import Qwen2Config, Qwen2ForCausalLM
    cfg = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=512, tie_word_embeddings=True,
               max_position_embeddings=512)
    hf = _init(Qwen2ForCausalLM(Qwen2Config(**cfg)))
    for n, p in hf.named_parameters():
        if n.endswith("bias"):
            p.data.normal_(0, 0.05)
    path = _save(str(tmp_path / "qwen2"), hf, cfg, "Qwen2ForCausalLM", "qwen2")
    assert _generate(path, PROMPTS) == _hf_generate(hf, PROMPTS)


def test_qwen3_moe_matches_hf_fused_and_per_expert_checkpoints(tmp_path):
    from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM
    cfg = dict(hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, rope_theta=1e6,
               vocab_size=512, num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1,
               mlp_only_layers=[], tie_word_embeddings=False, max_position_embeddings=512)
    hf = _init(Qwen3MoeForCausalLM(Qwen3MoeConfig(**cfg)))
    want = _hf_generate(hf, PROMPTS)
    fused = _save(str(tmp_path / "moe_fused"), hf, cfg, "Qwen3MoeForCausalLM", "qwen3_moe")
    assert _generate(fused, PROMPTS) == want

    def per_expert(sd):
        out = {}
        for k, v in sd.items():
            if k.endswith("mlp.experts.gate_up_proj"):
                base = k[: -len("gate_up_proj")]
                I = v.shape[1] // 2
                for e in range(v.shape[0]):
                    out[f"{base}{e}.gate_proj.weight"] = v[e, :I].contiguous()
                    out[f"{base}{e}.up_proj.weight"] = v[e, I:].contiguous()
            elif k.endswith("mlp.experts.down_proj"):
                base = k[: -len("down_proj")]
                for e in range(v.shape[0]):
                    out[f"{base}{e}.down_proj.weight"] = v[e].contiguous()
            else:
                out[k] = v
        return out

    hub = _save(str(tmp_path / "moe_hub"), hf, cfg, "Qwen3MoeForCausalLM", "qwen3_moe", rename=per_expert)
    assert _generate(hub, PROMPTS) == want


def test_missing_parameter_is_an_error(tmp_path):
    from transformers import Qwen3Config, Qwen3ForCausalLM
    cfg = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=2,
               num_key_value_heads=2, head_dim=32, vocab_size=128, tie_word_embeddings=False)
    hf = _init(Qwen3ForCausalLM(Qwen3Config(**cfg)))
    path = _save(str(tmp_path / "broken"), hf, cfg, "Qwen3ForCausalLM", "qwen3",
                 rename=lambda sd: {k: v for k, v in sd.items() if "down_proj" not in k})
    with pytest.raises(RuntimeError, match="missing"):
        _generate(path, PROMPTS[:1], n=1)


def test_deepseek_v3_mla_moe_matches_hf(tmp_path):
    from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
    cfg = dict(hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=3,
               num_attention_heads=4, num_key_value_heads=4, q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=32,
               qk_rope_head_dim=16, v_head_dim=32, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=3,
               n_group=4, topk_group=2, scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True,
               routed_scaling_factor=2.5, first_k_dense_replace=1, moe_layer_freq=1, rms_norm_eps=1e-6,
               rope_theta=10000.0, vocab_size=512, tie_word_embeddings=False, max_position_embeddings=512,
               rope_scaling=None, attention_bias=False)
    hf = _init(DeepseekV3ForCausalLM(DeepseekV3Config(**cfg)))
    for n, b in hf.named_buffers():
        if "e_score_correction_bias" in n:
            b.data.normal_(0, 0.1)
    for n, p in hf.named_parameters():
        if "e_score_correction_bias" in n:
            p.data.normal_(0, 0.1)
    path = _save(str(tmp_path / "dsv3"), hf, cfg, "DeepseekV3ForCausalLM", "deepseek_v3")
    assert _generate(path, PROMPTS, n=8) == _hf_generate(hf, PROMPTS, n=8)


@pytest.mark.parametrize("hybrid", [True, False])
def test_gemma2_sliding_window_softcap_matches_hf(tmp_path, hybrid):
    """Alternating sliding/global layers through the dual KV pool, the SWA allocator and the
    window-aware radix cache (`hybrid`), or a single pool (`disable_hybrid_swa_memory`)."""
    from transformers import Gemma2Config, Gemma2ForCausalLM
    cfg = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
               num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=512,
               tie_word_embeddings=True, max_position_embeddings=512, sliding_window=16, query_pre_attn_scalar=32,
               attn_logit_softcapping=50.0, final_logit_softcapping=30.0, hidden_activation="gelu_pytorch_tanh")
    hf = _init(Gemma2ForCausalLM(Gemma2Config(**cfg, attn_implementation="eager")))
    path = _save(str(tmp_path / "gemma2"), hf, cfg, "Gemma2ForCausalLM", "gemma2")
    prompts = [list(range(5, 60)), [9, 8, 7, 6, 5, 4, 3] * 5, [100, 200, 300]]
    want = _hf_generate(hf, prompts, n=12)
    got = _generate(path, prompts, n=12, disable_hybrid_swa_memory=not hybrid)
    assert got == want
    # a second pass reuses cached prefixes (window-aware matching) and must not change the result
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    ps.reset_state()
    eng = Engine(model_path=path, device="cpu", dtype="float32", page_size=4, skip_tokenizer_init=True,
                 max_total_tokens=1024, enable_single_process=True, disable_hybrid_swa_memory=not hybrid)
    try:
        sp = {"max_new_tokens": 12, "temperature": 0, "ignore_eos": True}
        first = [o["output_ids"] for o in eng.generate(input_ids=prompts, sampling_params=sp)]
        second = eng.generate(input_ids=prompts, sampling_params=sp)
        assert first == want and [o["output_ids"] for o in second] == want
        assert second[0]["meta_info"]["cached_tokens"] > 0
    finally:
        eng.shutdown()


def test_glm4_moe_matches_hf(tmp_path):
    from transformers import Glm4MoeConfig, Glm4MoeForCausalLM
    cfg = dict(hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=3,
               num_attention_heads=4, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5, rope_theta=10000.0,
               vocab_size=512, tie_word_embeddings=False, max_position_embeddings=512, partial_rotary_factor=0.5,
               n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, n_group=2, topk_group=1,
               routed_scaling_factor=1.5, norm_topk_prob=True, first_k_dense_replace=1, use_qk_norm=True,
               attention_bias=True)
    hf = _init(Glm4MoeForCausalLM(Glm4MoeConfig(**cfg)))
    for n, p in hf.named_parameters():
        if n.endswith("bias") and p.dim() == 1:
            p.data.normal_(0, 0.05)
    for n, b in hf.named_buffers():
        if "e_score_correction_bias" in n:
            b.data.normal_(0, 0.1)
    path = _save(str(tmp_path / "glm4moe"), hf, cfg, "Glm4MoeForCausalLM", "glm4_moe")
    assert _generate(path, PROMPTS) == _hf_generate(hf, PROMPTS)


def test_minimax_m2_matches_hf(tmp_path):
    from transformers import MiniMaxM2Config, MiniMaxM2ForCausalLM
    cfg = dict(hidden_size=128, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, vocab_size=512, tie_word_embeddings=False,
               max_position_embeddings=512, num_local_experts=8, num_experts_per_tok=2,
               rope_parameters={"rope_theta": 10000.0, "rope_type": "default"})
    hf = _init(MiniMaxM2ForCausalLM(MiniMaxM2Config(**cfg)))
    for n, b in hf.named_buffers():
        if "e_score_correction_bias" in n:
            b.data.normal_(0, 0.1)
    for n, p in hf.named_parameters():
        if "q_norm" in n or "k_norm" in n:
            p.data.uniform_(0.5, 1.5)
    path = _save(str(tmp_path / "m2"), hf, dict(cfg, rope_theta=10000.0), "MiniMaxM2ForCausalLM", "minimax_m2")
    assert _generate(path, PROMPTS) == _hf_generate(hf, PROMPTS)


def _dense_reference_generate(step_logits, prompts, n):
    """Greedy decoding with a plain full-sequence forward (no KV cache) as the oracle."""
    outs = []
    for p in prompts:
        ids = list(p)
        for _ in range(n):
            ids.append(int(step_logits(torch.tensor(ids))[-1].argmax()))
        outs.append(ids[len(p):])
    return outs


def test_grok_matches_plain_torch_restatement(tmp_path):
    """No HF class exists for Grok: the oracle is a direct restatement of the layer math in
    plain torch over the same random checkpoint."""
    import math
    from safetensors.torch import save_file
    torch.manual_seed(0)
    H, I, nh, nkv, D, V, L, E, K = 64, 96, 4, 2, 16, 128, 2, 4, 2
    cfg = dict(architectures=["Grok1ForCausalLM"], model_type="grok-1", hidden_size=H, intermediate_size=I,
               moe_intermediate_size=I, num_hidden_layers=L, num_attention_heads=nh, num_key_value_heads=nkv,
               head_dim=D, rms_norm_eps=1e-5, rope_theta=10000, vocab_size=V, max_position_embeddings=256,
               num_local_experts=E, num_experts_per_tok=K, attn_logit_softcapping=30.0, router_logit_softcapping=30.0,
               final_logit_softcapping=0.0, embedding_multiplier_scale=3.0, output_multiplier_scale=0.5,
               residual_moe=True, torch_dtype="float32", tie_word_embeddings=False)
    sd = {"model.embed_tokens.weight": torch.randn(V, H) * 0.3, "lm_head.weight": torch.randn(V, H) * 0.3,
          "model.norm.weight": torch.rand(H) + 0.5}
    for i in range(L):
        p = f"model.layers.{i}."
        sd[p + "self_attn.q_proj.weight"] = torch.randn(nh * D, H) * 0.2
        sd[p + "self_attn.k_proj.weight"] = torch.randn(nkv * D, H) * 0.2
        sd[p + "self_attn.v_proj.weight"] = torch.randn(nkv * D, H) * 0.2
        sd[p + "self_attn.o_proj.weight"] = torch.randn(H, nh * D) * 0.2
        for nm in ("pre_attn_norm", "post_attn_norm", "pre_moe_norm", "post_moe_norm"):
            sd[p + nm + ".weight"] = torch.rand(H) + 0.5
        sd[p + "block_sparse_moe.gate.weight"] = torch.randn(E, H)
        for e in range(E):
            sd[p + f"block_sparse_moe.experts.{e}.w1.weight"] = torch.randn(I, H) * 0.2
            sd[p + f"block_sparse_moe.experts.{e}.w3.weight"] = torch.randn(I, H) * 0.2
            sd[p + f"block_sparse_moe.experts.{e}.w2.weight"] = torch.randn(H, I) * 0.2
        sd[p + "mlp.gate_proj.weight"] = torch.randn(I, H) * 0.2
        sd[p + "mlp.up_proj.weight"] = torch.randn(I, H) * 0.2
        sd[p + "mlp.down_proj.weight"] = torch.randn(H, I) * 0.2
    path = str(tmp_path / "grok")
    os.makedirs(path)
    save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w

    def rope(x, pos):
        half = D // 2
        inv = 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D))
        ang = pos[:, None].float() * inv[None]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    gelu = lambda t: torch.nn.functional.gelu(t, approximate="tanh")

    def logits_of(ids):
        T = len(ids)
        pos = torch.arange(T)
        x = sd["model.embed_tokens.weight"][ids] * 3.0
        for i in range(L):
            p = f"model.layers.{i}."
            h = rms(x, sd[p + "pre_attn_norm.weight"])
            q = rope((h @ sd[p + "self_attn.q_proj.weight"].T).view(T, nh, D), pos)
            k = rope((h @ sd[p + "self_attn.k_proj.weight"].T).view(T, nkv, D), pos)
            v = (h @ sd[p + "self_attn.v_proj.weight"].T).view(T, nkv, D)
            k, v = k.repeat_interleave(nh // nkv, 1), v.repeat_interleave(nh // nkv, 1)
            s = torch.einsum("qhd,khd->hqk", q, k) * D ** -0.5
            s = 30.0 * torch.tanh(s / 30.0)
            s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(T, nh * D)
            x = x + rms(a @ sd[p + "self_attn.o_proj.weight"].T, sd[p + "post_attn_norm.weight"])
            h = rms(x, sd[p + "pre_moe_norm.weight"])
            rl = h @ sd[p + "block_sparse_moe.gate.weight"].T
            rl = 30.0 * torch.tanh(rl / 30.0)
            w, idx = torch.topk(torch.softmax(rl, -1), K, -1)
            y = torch.zeros_like(h)
            for t in range(T):
                for j in range(K):
                    e = int(idx[t, j])
                    pe = p + f"block_sparse_moe.experts.{e}."
                    y[t] += w[t, j] * ((gelu(h[t] @ sd[pe + "w1.weight"].T) * (h[t] @ sd[pe + "w3.weight"].T)) @ sd[pe + "w2.weight"].T)
            d = (gelu(h @ sd[p + "mlp.gate_proj.weight"].T) * (h @ sd[p + "mlp.up_proj.weight"].T)) @ sd[p + "mlp.down_proj.weight"].T
            x = x + rms((y + d) / math.sqrt(2.0), sd[p + "post_moe_norm.weight"])
        return (rms(x, sd["model.norm.weight"]) @ sd["lm_head.weight"].T) * 0.5

    prompts = [[5, 9, 33, 7, 100, 2], [1, 2, 3]]
    want = _dense_reference_generate(logits_of, prompts, 6)
    assert _generate(path, prompts, n=6) == want


def test_bailing_moe_is_glm4_moe_under_other_names(tmp_path):
    """Ling checkpoints (fused `query_key_value`, `word_embeddings`, `expert_bias`) must produce
    what the equivalent GLM-4-MoE checkpoint produces (which is checked against HF above)."""
    from transformers import Glm4MoeConfig, Glm4MoeForCausalLM
    cfg = dict(hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=3,
               num_attention_heads=4, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5, rope_theta=10000.0,
               vocab_size=512, tie_word_embeddings=False, max_position_embeddings=512, partial_rotary_factor=0.5,
               n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, n_group=2, topk_group=1,
               routed_scaling_factor=1.5, norm_topk_prob=True, first_k_dense_replace=1, use_qk_norm=True,
               attention_bias=False)
    hf = _init(Glm4MoeForCausalLM(Glm4MoeConfig(**cfg)))
    for n, b in hf.named_buffers():
        if "e_score_correction_bias" in n:
            b.data.normal_(0, 0.1)
    want = _hf_generate(hf, PROMPTS)

    def rename(sd):
        out = {}
        qkv = {}
        for k, v in sd.items():
            k = k.replace("model.embed_tokens.", "model.word_embeddings.").replace(".self_attn.o_proj.", ".attention.dense.")
            k = k.replace(".self_attn.q_norm.", ".attention.query_layernorm.").replace(".self_attn.k_norm.", ".attention.key_layernorm.")
            k = k.replace(".mlp.gate.e_score_correction_bias", ".mlp.gate.expert_bias")
            for p in ("q_proj", "k_proj", "v_proj"):
                if f".self_attn.{p}.weight" in k:
                    qkv.setdefault(k.split(".self_attn.")[0], {})[p] = v
                    break
            else:
                out[k] = v
        for head, d in qkv.items():
            out[head + ".attention.query_key_value.weight"] = torch.cat([d["q_proj"], d["k_proj"], d["v_proj"]], 0)
        return out

    ling = dict(cfg, num_experts=8, num_shared_experts=1, score_function="sigmoid", moe_router_enable_expert_bias=True)
    for k in ("n_routed_experts", "n_shared_experts"):
        ling.pop(k)
    path = _save(str(tmp_path / "ling"), hf, ling, "BailingMoeV2ForCausalLM", "bailing_moe", rename=rename)
    assert _generate(path, PROMPTS) == want


@pytest.mark.parametrize("moe", [True, False])
def test_qwen3_next_hybrid_gated_deltanet_matches_hf(tmp_path, moe):
    """Linear-attention layers over the recurrent state pool (chunked prefill + recurrent decode,
    state carried across prefill chunks) interleaved with gated softmax attention."""
    from transformers import Qwen3NextConfig, Qwen3NextForCausalLM
    cfg = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
               num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, vocab_size=512, tie_word_embeddings=False,
               max_position_embeddings=512, partial_rotary_factor=0.25, linear_num_value_heads=4,
               linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4,
               num_experts=8 if moe else 0, num_experts_per_tok=2, moe_intermediate_size=64,
               shared_expert_intermediate_size=64, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[],
               layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
               rope_parameters={"rope_theta": 10000.0, "rope_type": "default", "partial_rotary_factor": 0.25})
    hf = _init(Qwen3NextForCausalLM(Qwen3NextConfig(**cfg)))
    for n, p in hf.named_parameters():
        if n.endswith("A_log"):
            p.data.uniform_(-1.0, 1.0)
        elif n.endswith("dt_bias"):
            p.data.uniform_(0.5, 1.5)
        elif "norm" in n:
            p.data.normal_(0, 0.1)
    path = _save(str(tmp_path / "q3n"), hf, dict(cfg, rope_theta=10000.0), "Qwen3NextForCausalLM", "qwen3_next")
    prompts = [list(range(5, 90)), [9, 8, 7, 6, 5, 4, 3] * 5, [100, 200, 300]]
    want = _hf_generate(hf, prompts, n=8)
    assert _generate(path, prompts, n=8) == want
    # prefill in chunks of 32 tokens: the conv window and the recurrent matrix cross chunk borders
    assert _generate(path, prompts, n=8, chunked_prefill_size=32) == want


@pytest.mark.parametrize("moe,wrapped", [(False, False), (True, False), (False, True)])
def test_qwen3_5_matches_hf(tmp_path, moe, wrapped):
    """Qwen3.5 (dense and MoE): the Gated DeltaNet input projection arrives as four tensors and is regrouped at load.
    `wrapped`: the layout of a `Qwen3_5ForConditionalGeneration` checkpoint (text model under
    `model.language_model.`, nested `text_config`, vision tower and MTP head present and skipped)."""
    import transformers
    cfg = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
               num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, vocab_size=512, tie_word_embeddings=False,
               max_position_embeddings=512, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16,
               linear_value_head_dim=16, linear_conv_kernel_dim=4,
               layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
               rope_parameters={"rope_theta": 10000.0, "rope_type": "default", "partial_rotary_factor": 0.25,
                                "mrope_section": [2, 1, 1], "mrope_interleaved": True})
    if moe:
        cfg.update(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=64)
        hf = _init(transformers.Qwen3_5MoeForCausalLM(transformers.Qwen3_5MoeTextConfig(**cfg)))
    else:
        hf = _init(transformers.Qwen3_5ForCausalLM(transformers.Qwen3_5TextConfig(**cfg)))
    for n, p in hf.named_parameters():
        if n.endswith("A_log"):
            p.data.uniform_(-1.0, 1.0)
        elif n.endswith("dt_bias"):
            p.data.uniform_(0.5, 1.5)
        elif "norm" in n:
            p.data.normal_(0, 0.1)
    text = dict(cfg, rope_theta=10000.0, partial_rotary_factor=0.25)
    if wrapped:
        def rename(sd):
            out = {k.replace("model.", "model.language_model.", 1) if k.startswith("model.") else k: v
                   for k, v in sd.items()}
            out["model.visual.patch_embed.proj.bias"] = torch.zeros(8)
            out["mtp.fc.weight"] = torch.zeros(4, 4)
            return out
        path = _save(str(tmp_path / "q35"), hf, dict(text_config=dict(text, model_type="qwen3_5_text"),
                                                     vision_config={"depth": 1}, tie_word_embeddings=False),
                     "Qwen3_5ForConditionalGeneration", "qwen3_5", rename=rename)
    else:
        path = _save(str(tmp_path / "q35"), hf, text, "Qwen3_5MoeForCausalLM" if moe else "Qwen3_5ForCausalLM",
                     "qwen3_5_moe_text" if moe else "qwen3_5_text")
    prompts = [list(range(5, 90)), [9, 8, 7, 6, 5, 4, 3] * 5, [100, 200, 300]]
    want = _hf_generate(hf, prompts, n=8)
    assert _generate(path, prompts, n=8) == want
    if not wrapped:
        assert _generate(path, prompts, n=8, chunked_prefill_size=32) == want


@pytest.mark.parametrize("kind", ["umt5", "t5"])
def test_t5_family_encoder_matches_hf(tmp_path, kind):
    import transformers
    from sglang_jax_b200.models.umt5 import T5EncoderModel, UMT5EncoderModel
    cfg_cls, hf_cls, mine = (transformers.UMT5Config, transformers.UMT5EncoderModel, UMT5EncoderModel) if kind == "umt5" \
        else (transformers.T5Config, transformers.T5EncoderModel, T5EncoderModel)
    cfg = cfg_cls(vocab_size=300, d_model=64, d_kv=16, d_ff=128, num_layers=3, num_heads=4,
                  relative_attention_num_buckets=32, relative_attention_max_distance=128,
                  feed_forward_proj="gated-gelu", dropout_rate=0.0)
    hf = _init(hf_cls(cfg), 0.1)
    model = mine(cfg, dtype=torch.float32)
    loaded = model.load_weights(hf.state_dict().items())
    assert loaded == {n for n, _ in model.named_parameters()}
    ids = torch.randint(0, 300, (2, 23), generator=torch.Generator().manual_seed(0))
    mask = torch.ones(2, 23, dtype=torch.long)
    mask[1, 17:] = 0
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask).last_hidden_state
    got = model.encode(ids, mask)
    assert torch.allclose(got[0], want[0], atol=2e-5) and torch.allclose(got[1, :17], want[1, :17], atol=2e-5)


@pytest.mark.parametrize("tied", [False, True])
def test_umt5_conditional_generation_matches_hf(tied):
    """Encoder-decoder UMT5: teacher-forced logits, the bare decoder / encoder-decoder classes and greedy generation
    with cached keys / values against HF `UMT5ForConditionalGeneration`."""
    import transformers
    from sglang_jax_b200.models.umt5 import UMT5DecoderModel, UMT5ForConditionalGeneration, UMT5Model
    cfg = transformers.UMT5Config(vocab_size=300, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_decoder_layers=3,
                                  num_heads=4, relative_attention_num_buckets=32, relative_attention_max_distance=128,
                                  feed_forward_proj="gated-gelu", dropout_rate=0.0, tie_word_embeddings=tied,
                                  decoder_start_token_id=0, pad_token_id=0, eos_token_id=1)
    hf = _init(transformers.UMT5ForConditionalGeneration(cfg), 0.1)
    if tied:
        hf.tie_weights()
    model = UMT5ForConditionalGeneration(cfg, dtype=torch.float32)
    loaded = model.load_weights(hf.state_dict().items())
    assert loaded == {n for n, _ in model.named_parameters()}
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(2, 300, (2, 19), generator=g)
    mask = torch.ones(2, 19, dtype=torch.long)
    mask[1, 13:] = 0
    dec = torch.randint(2, 300, (2, 9), generator=g)
    dec[:, 0] = 0
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=mask, decoder_input_ids=dec, output_hidden_states=True,
                 use_cache=False)
    got = model(ids, dec, mask)
    assert torch.allclose(got, ref.logits, atol=1e-4), (got - ref.logits).abs().max()
    # the head-less classes load the same checkpoint and give the decoder's last hidden state
    plain = UMT5Model(cfg, dtype=torch.float32)
    plain.load_weights(hf.state_dict().items())
    hid = plain(ids, dec, mask)
    assert torch.allclose(hid, ref.decoder_hidden_states[-1], atol=1e-4)
    only = UMT5DecoderModel(cfg, dtype=torch.float32)
    assert only.load_weights(hf.state_dict().items()) == {n for n, _ in only.named_parameters()}
    assert torch.allclose(only(dec, ref.encoder_last_hidden_state, mask), hid, atol=1e-4)
    # greedy generation with the incremental cache == HF generate
    with torch.no_grad():
        want = hf.generate(input_ids=ids, attention_mask=mask, max_new_tokens=8, do_sample=False, num_beams=1,
                           use_cache=False)
    mine = model.generate(ids, max_new_tokens=8, attention_mask=mask)
    want = want[:, 1:]                                   # HF returns the start token first
    n = min(want.shape[1], mine.shape[1])
    assert n >= 1 and torch.equal(mine[:, :n], want[:, :n])


def _run_dummy(cfg: dict, tmp_path, name: str, prompts, n=6, **kw):
    """Random-weight model: outputs must not depend on how the prompt was chunked or batched
    (state hand-over between chunks / decode steps is exact) and must be deterministic."""
    path = str(tmp_path / name)
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(dict(cfg, torch_dtype="float32"), f)
    a = _generate(path, prompts, n=n, load_format="dummy", **kw)
    b = _generate(path, prompts, n=n, load_format="dummy", chunked_prefill_size=32, **kw)
    c = [_generate(path, [p], n=n, load_format="dummy", **kw)[0] for p in prompts]
    assert a == b == c, (a, b, c)
    assert len({t for o in a for t in o}) > 2, a          # a collapsed model would pass the invariance trivially
    return a


def test_kimi_linear_kda_hybrid_is_chunk_and_batch_invariant(tmp_path):
    cfg = dict(architectures=["KimiLinearForCausalLM"], model_type="kimi_linear", hidden_size=64, intermediate_size=96,
               moe_intermediate_size=32, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=4,
               rms_norm_eps=1e-5, vocab_size=256, max_position_embeddings=512, kv_lora_rank=32, q_lora_rank=None,
               qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, mla_use_nope=True, num_experts=4,
               num_experts_per_token=2, num_shared_experts=1, first_k_dense_replace=1, moe_layer_freq=1,
               moe_router_activation_func="sigmoid", routed_scaling_factor=1.0, tie_word_embeddings=False,
               linear_attn_config={"kda_layers": [1, 2, 3], "full_attn_layers": [4], "num_heads": 4, "head_dim": 16,
                                   "short_conv_kernel_size": 4})
    out = _run_dummy(cfg, tmp_path, "kimi", [list(range(5, 80)), [9, 8, 7, 6] * 3])
    assert all(len(o) == 6 for o in out)


def test_bailing_linear_lightning_hybrid_is_chunk_and_batch_invariant(tmp_path):
    cfg = dict(architectures=["BailingMoeLinearForCausalLM"], model_type="bailing_moe_linear", hidden_size=64,
               intermediate_size=96, moe_intermediate_size=32, num_hidden_layers=4, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-5, vocab_size=256, max_position_embeddings=512,
               num_experts=4, num_experts_per_tok=2, num_shared_experts=1, first_k_dense_replace=1, n_group=1,
               topk_group=1, routed_scaling_factor=1.0, score_function="sigmoid", layer_group_size=4,
               tie_word_embeddings=False, rope_theta=10000.0, partial_rotary_factor=0.5)
    out = _run_dummy(cfg, tmp_path, "lingl", [list(range(5, 80)), [9, 8, 7, 6] * 3])
    assert all(len(o) == 6 for o in out)


@pytest.mark.parametrize("family", ["kimi_linear", "bailing_linear"])
def test_kda_and_lightning_hybrids_share_prefixes_through_page_checkpoints(tmp_path, family):
    """Pages of 16 tokens and chunked prefill: the recurrent state is checkpointed at the last page boundary inside
    each prefill step, a later request with the same opening restarts from that checkpoint (KV reused, state cloned)
    and generates exactly what it generates without any sharing."""
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    if family == "kimi_linear":
        cfg = dict(architectures=["KimiLinearForCausalLM"], model_type="kimi_linear", hidden_size=64,
                   intermediate_size=96, moe_intermediate_size=32, num_hidden_layers=4, num_attention_heads=4,
                   num_key_value_heads=4, rms_norm_eps=1e-5, vocab_size=256, max_position_embeddings=512,
                   kv_lora_rank=32, q_lora_rank=None, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                   mla_use_nope=True, num_experts=4, num_experts_per_token=2, num_shared_experts=1,
                   first_k_dense_replace=1, moe_layer_freq=1, moe_router_activation_func="sigmoid",
                   routed_scaling_factor=1.0, tie_word_embeddings=False,
                   linear_attn_config={"kda_layers": [1, 2, 3], "full_attn_layers": [4], "num_heads": 4,
                                       "head_dim": 16, "short_conv_kernel_size": 4})
    else:
        cfg = dict(architectures=["BailingMoeLinearForCausalLM"], model_type="bailing_moe_linear", hidden_size=64,
                   intermediate_size=96, moe_intermediate_size=32, num_hidden_layers=4, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-5, vocab_size=256, max_position_embeddings=512,
                   num_experts=4, num_experts_per_tok=2, num_shared_experts=1, first_k_dense_replace=1, n_group=1,
                   topk_group=1, routed_scaling_factor=1.0, score_function="sigmoid", layer_group_size=4,
                   tie_word_embeddings=False, rope_theta=10000.0, partial_rotary_factor=0.5)
    path = tmp_path / family
    path.mkdir()
    (path / "config.json").write_text(json.dumps(dict(cfg, torch_dtype="float32")))
    opening = list(range(5, 75))                                 # 70 tokens: page boundaries at 16 .. 64
    sp = {"max_new_tokens": 5, "temperature": 0, "ignore_eos": True}

    def run(**kw):
        ps.reset_state()
        eng = Engine(model_path=str(path), device="cpu", dtype="float32", page_size=16, skip_tokenizer_init=True,
                     max_total_tokens=2048, enable_single_process=True, load_format="dummy", chunked_prefill_size=32,
                     **kw)
        try:
            a = eng.generate(input_ids=opening + [200, 201], sampling_params=sp)
            b = eng.generate(input_ids=[opening + [210, 211, 212], opening[:40] + [99] * 9], sampling_params=sp)
            tc = eng.scheduler.tree_cache
            if hasattr(tc, "assert_recurrent_slot_ledger"):
                tc.assert_recurrent_slot_ledger()
            eng.scheduler.check_memory()
            return (type(tc).__name__, a["output_ids"], [o["output_ids"] for o in b],
                    [o["meta_info"]["cached_tokens"] for o in b])
        finally:
            eng.shutdown()

    shared, plain = run(), run(disable_radix_cache=True)
    assert shared[0] == "UnifiedRadixCache"
    assert shared[1:3] == plain[1:3]
    assert len({t for o in shared[2] for t in o}) > 2
    assert shared[3] == [64, 32] and plain[3] == [0, 0]          # checkpoints at the chunk ends 32 and 64
    coarse = run(recurrent_track_interval=32)                    # checkpoints only on multiples of 32 tokens
    assert coarse[1:3] == plain[1:3] and coarse[3] == [64, 32]
    with pytest.raises(Exception):
        run(recurrent_track_interval=24)                         # not a multiple of the page size


def test_kda_and_lightning_ops_match_stepwise_recurrence():
    from sglang_jax_b200.ops import linear_attention as la
    g = torch.Generator().manual_seed(0)
    B, T, H, D = 2, 9, 3, 8
    q, k, v = (torch.randn(B, T, H, D, generator=g) for _ in range(3))
    gate = -torch.rand(B, T, H, D, generator=g)
    beta = torch.rand(B, T, H, generator=g)
    S0 = torch.randn(B, H, D, D, generator=g) * 0.1
    o_all, S_all = la.kda_recurrent(q, k, v, gate, beta, S0)
    S, outs = S0, []
    for t in range(T):                       # one step at a time == all steps at once
        o, S = la.kda_recurrent(q[:, t:t + 1], k[:, t:t + 1], v[:, t:t + 1], gate[:, t:t + 1], beta[:, t:t + 1], S)
        outs.append(o)
    assert torch.allclose(torch.cat(outs, 1), o_all, atol=1e-5) and torch.allclose(S, S_all, atol=1e-5)
    # with a zero gate and beta = 1 the delta rule stores exact key -> value associations
    kk = torch.nn.functional.normalize(torch.eye(D)[None, :3, None, :].expand(1, 3, 1, D), dim=-1)
    vv = torch.randn(1, 3, 1, D, generator=g)
    _, S = la.kda_recurrent(kk, kk, vv, torch.zeros(1, 3, 1, D), torch.ones(1, 3, 1), torch.zeros(1, 1, D, D))
    assert torch.allclose((S[0, 0] * kk[0, 1, 0].unsqueeze(-1)).sum(0), vv[0, 1, 0], atol=1e-5)
    slopes = la.alibi_slopes(H)
    o_all, S_all = la.lightning_attention(q, k, v, slopes, S0)
    o1, S1 = la.lightning_attention(q[:, :4], k[:, :4], v[:, :4], slopes, S0)
    o2, S2 = la.lightning_attention(q[:, 4:], k[:, 4:], v[:, 4:], slopes, S1)
    assert torch.allclose(torch.cat([o1, o2], 1), o_all, atol=1e-5) and torch.allclose(S2, S_all, atol=1e-5)
    assert la.alibi_slopes(6).shape == (6,)


def test_mimo_v2_flash_hybrid_swa_sinks_and_narrow_values(tmp_path):
    cfg = dict(architectures=["MiMoV2FlashForCausalLM"], model_type="mimo_v2_flash", hidden_size=64,
               intermediate_size=96, moe_intermediate_size=32, num_hidden_layers=4, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, v_head_dim=8, swa_num_attention_heads=4, swa_num_key_value_heads=4,
               swa_head_dim=16, swa_v_head_dim=8, swa_rope_theta=10000.0, rope_theta=1000000.0,
               sliding_window_size=24, hybrid_layer_pattern=[0, 1, 1, 0], moe_layer_freq=[0, 1, 1, 1],
               add_swa_attention_sink_bias=True, add_full_attention_sink_bias=False, attention_value_scale=0.7,
               partial_rotary_factor=0.5, n_routed_experts=4, num_experts_per_tok=2, scoring_func="sigmoid",
               topk_method="noaux_tc", norm_topk_prob=True, layernorm_epsilon=1e-5, vocab_size=256,
               max_position_embeddings=512, tie_word_embeddings=False)
    out = _run_dummy(cfg, tmp_path, "mimo2", [list(range(5, 80)), [9, 8, 7, 6] * 3])
    assert all(len(o) == 6 for o in out)
    from sglang_jax_b200.models.mimo_v2_flash import MiMoV2FlashForCausalLM
    from types import SimpleNamespace
    m = MiMoV2FlashForCausalLM(SimpleNamespace(**cfg), dtype=torch.float32)
    assert m.swa_layer_ids == [1, 2] and m.swa_kv_shape == (4, 16)
    assert m.model.layers[1].self_attn.attention_sink_bias is not None
    assert m.model.layers[0].self_attn.attention_sink_bias is None
    assert m.model.layers[0].self_attn.o_proj.weight.shape[1] == 4 * 8


def test_mimo_v2_pro_fused_qkv_checkpoints_bf16_and_per_shard_fp8():
    """MiMo-V2-Pro stores the attention input projection fused.  bf16: rows are [Q | K | V].  Block-FP8: quantised per
    tensor shard and concatenated, so every shard is de-quantised on its own block grid (a scale block straddles the
    K / V border inside a shard) before Q / K / V are regrouped.  Both must fill the fused parameter exactly like the
    Flash layout with separate projections does."""
    from types import SimpleNamespace
    from sglang_jax_b200.models.mimo_v2_flash import (MiMoV2FlashForCausalLM, MiMoV2ForCausalLM, infer_qkv_shards)
    from sglang_jax_b200.model_loader.loader import dequant_static_fp8
    from sglang_jax_b200.models.registry import get_model_class
    cfg = dict(hidden_size=256, intermediate_size=96, moe_intermediate_size=32, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, head_dim=64, v_head_dim=32, swa_num_attention_heads=4,
               swa_num_key_value_heads=2, swa_head_dim=64, swa_v_head_dim=32, rope_theta=1e6, sliding_window_size=24,
               hybrid_layer_pattern=[0, 1], moe_layer_freq=[0, 0], add_swa_attention_sink_bias=False,
               add_full_attention_sink_bias=False, partial_rotary_factor=0.5, n_routed_experts=0,
               num_experts_per_tok=2, layernorm_epsilon=1e-5, vocab_size=64, max_position_embeddings=128,
               tie_word_embeddings=False, quantization_config={"weight_block_size": [128, 128]})
    assert get_model_class(["MiMoV2ForCausalLM"]) is MiMoV2ForCausalLM
    g = torch.Generator().manual_seed(0)
    nh, nkv, hd, vd, H = 4, 2, 64, 32, 256
    qkv = {i: [torch.randn(n, H, generator=g) * 0.05 for n in (nh * hd, nkv * hd, nkv * vd)] for i in range(2)}

    def flash_names(tensors):
        for i, (q, k, v) in tensors.items():
            for n, w in (("q_proj", q), ("k_proj", k), ("v_proj", v)):
                yield f"model.layers.{i}.self_attn.{n}.weight", w

    def fused_param(model, i):
        return model.model.layers[i].self_attn.qkv_proj.weight.clone()

    want = MiMoV2FlashForCausalLM(SimpleNamespace(**cfg), dtype=torch.float32)
    want.load_weights(flash_names(qkv))
    # bf16 layout
    pro = MiMoV2ForCausalLM(SimpleNamespace(**cfg), dtype=torch.float32)
    pro.load_weights(pro.preprocess_checkpoint(
        (f"model.layers.{i}.self_attn.qkv_proj.weight", torch.cat(t, 0)) for i, t in qkv.items()))
    for i in range(2):
        assert torch.equal(fused_param(pro, i), fused_param(want, i))
    # block-FP8, two shards of 128 + 64 + 32 = 224 rows: the second scale block of a shard covers K and V rows
    tp, blk = 2, 128
    assert infer_qkv_shards(448, 4, nh, nkv, hd, vd, blk) == (2, 2)
    assert infer_qkv_shards(448, 4, nh, 4, hd, vd, blk) == (2, 2)          # config lists replicated KV heads
    names, deq = [], {}
    for i, (q, k, v) in qkv.items():
        ws, ss, dq = [], [], ([], [], [])
        for s in range(tp):
            shard = torch.cat([q.chunk(tp)[s], k.chunk(tp)[s], v.chunk(tp)[s]], 0)          # [224, 256]
            pad = torch.zeros(256, H)
            pad[:224] = shard
            blocks = pad.view(2, blk, 2, blk)
            scale = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-8) / 448.0                    # [2, 2]
            wq = (blocks / scale[:, None, :, None]).to(torch.float8_e4m3fn)
            back = (wq.float() * scale[:, None, :, None]).view(256, H)[:224]
            ws.append(wq.view(256, H)[:224])
            ss.append(scale)
            for dst, piece in zip(dq, torch.split(back, [128, 64, 32], 0)):
                dst.append(piece)
        names.append((f"model.layers.{i}.self_attn.qkv_proj.weight_scale_inv", torch.cat(ss, 0)))
        names.append((f"model.layers.{i}.self_attn.qkv_proj.weight", torch.cat(ws, 0)))
        deq[i] = [torch.cat(p, 0) for p in dq]
    want8 = MiMoV2FlashForCausalLM(SimpleNamespace(**cfg), dtype=torch.float32)
    want8.load_weights(flash_names(deq))
    pro8 = MiMoV2ForCausalLM(SimpleNamespace(**cfg), dtype=torch.float32)
    pro8.load_weights(dequant_static_fp8(pro8.preprocess_checkpoint(iter(names)), (128, 128)))
    for i in range(2):
        assert torch.equal(fused_param(pro8, i), fused_param(want8, i))
        assert not torch.equal(fused_param(pro8, i), fused_param(want, i))                   # it really was quantised


@pytest.mark.parametrize("moe", [False, True])
def test_gemma4_text_matches_hf(tmp_path, moe):
    """Sliding layers (narrow heads, plain RoPE) and global layers (wide heads, proportional RoPE,
    values taken from the key projection), scale-free V norm, optional routed GeGLU block."""
    from transformers.models.gemma4 import Gemma4ForCausalLM, Gemma4TextConfig
    cfg = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, global_head_dim=32, num_global_key_value_heads=1,
               attention_k_eq_v=True, rms_norm_eps=1e-6, vocab_size=300, tie_word_embeddings=True,
               max_position_embeddings=512, sliding_window=16, final_logit_softcapping=30.0,
               hidden_activation="gelu_pytorch_tanh", hidden_size_per_layer_input=0, num_kv_shared_layers=0,
               layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
               vocab_size_per_layer_input=300)
    if moe:
        cfg.update(enable_moe_block=True, num_experts=4, top_k_experts=2, moe_intermediate_size=32)
    hf = _init(Gemma4ForCausalLM(Gemma4TextConfig(**cfg, attn_implementation="eager")))
    g = torch.Generator().manual_seed(1)
    for n, b in list(hf.named_buffers()):
        if n.endswith("layer_scalar"):
            b.copy_(0.5 + torch.rand(1, generator=g))
    for n, p in hf.named_parameters():
        if n.endswith("per_expert_scale") or n.endswith("router.scale"):
            p.data.copy_(0.5 + torch.rand(p.shape, generator=g))
    full_cfg = Gemma4TextConfig(**cfg).to_dict()
    full_cfg.pop("architectures", None)
    path = _save(str(tmp_path / "gemma4"), hf, full_cfg, "Gemma4ForCausalLM", "gemma4_text")
    prompts = [list(range(5, 60)), [9, 8, 7, 6, 5, 4, 3] * 5, [100, 200, 250]]
    want = _hf_generate(hf, prompts, n=10)
    assert len({t for w in want for t in w}) > 4               # not a collapsed model: the comparison means something
    assert _generate(path, prompts, n=10) == want
    assert _generate(path, prompts, n=10, chunked_prefill_size=16) == want


@pytest.mark.parametrize("topk", [8, 4096])
def test_glm5_dsa_sparse_attention_matches_hf(tmp_path, topk):
    """GLM-5: latent attention whose keys are picked by the per-layer indexer.  `topk=8` makes the
    selection bite on every prompt longer than 8 tokens; `topk=4096` is the dense regime."""
    from transformers.models.glm_moe_dsa import GlmMoeDsaConfig, GlmMoeDsaForCausalLM
    cfg = dict(hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=3,
               num_attention_heads=4, num_key_value_heads=4, q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=32,
               qk_rope_head_dim=16, v_head_dim=32, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=3,
               n_group=1, topk_group=1, norm_topk_prob=True, routed_scaling_factor=2.5,
               mlp_layer_types=["dense", "sparse", "sparse"], rms_norm_eps=1e-6, vocab_size=512,
               tie_word_embeddings=False, max_position_embeddings=512, attention_bias=False,
               index_topk=topk, index_head_dim=32, index_n_heads=4,
               rope_parameters={"rope_type": "default", "rope_theta": 10000.0})
    hf = _init(GlmMoeDsaForCausalLM(GlmMoeDsaConfig(**cfg, attn_implementation="eager")))
    for n, b in hf.named_buffers():
        if "e_score_correction_bias" in n:
            b.data.normal_(0, 0.1)
    for n, p in hf.named_parameters():
        if n.endswith("k_norm.bias"):
            p.data.normal_(0, 0.1)
    # the HF port rotates split-half lanes in the main attention; released checkpoints interleave
    path = _save(str(tmp_path / "glm5"), hf, dict(cfg, rope_interleave=False), "GlmMoeDsaForCausalLM", "glm_moe_dsa")
    want = _hf_generate(hf, PROMPTS, n=8)
    assert len({t for w in want for t in w}) > 4
    assert _generate(path, PROMPTS, n=8) == want
    assert _generate(path, PROMPTS, n=8, chunked_prefill_size=16) == want


def test_kimi_k25_language_model_loads_under_language_model_prefix(tmp_path):
    """The checkpoint nests the DeepSeek-V3 decoder under `language_model.` beside the vision tower."""
    from safetensors.torch import save_file
    from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
    text = dict(hidden_size=128, intermediate_size=256, moe_intermediate_size=64, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=4, q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=32,
                qk_rope_head_dim=16, v_head_dim=32, n_routed_experts=4, n_shared_experts=1, num_experts_per_tok=2,
                n_group=1, topk_group=1, scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True,
                routed_scaling_factor=2.5, first_k_dense_replace=1, moe_layer_freq=1, rms_norm_eps=1e-6,
                rope_theta=10000.0, vocab_size=512, tie_word_embeddings=False, max_position_embeddings=512,
                rope_scaling=None, attention_bias=False)
    hf = _init(DeepseekV3ForCausalLM(DeepseekV3Config(**text)))
    path = tmp_path / "k25"
    path.mkdir()
    sd = {"language_model." + k: v.contiguous() for k, v in hf.state_dict().items()}
    sd["vision_tower.patch_embed.proj.bias"] = torch.zeros(8)
    sd["mm_projector.proj.0.bias"] = torch.zeros(8)
    save_file(sd, str(path / "model.safetensors"))
    cfg = dict(architectures=["KimiK25ForConditionalGeneration"], model_type="kimi_k25", torch_dtype="float32",
               text_config=dict(text, model_type="deepseek_v3", quantization_config={"format": "pack-quantized"}),
               vision_config={"vt_hidden_size": 8}, media_placeholder_token_id=500)
    (path / "config.json").write_text(json.dumps(cfg))
    assert _generate(str(path), PROMPTS, n=6) == _hf_generate(hf, PROMPTS, n=6)


def test_hybrid_recurrent_prefix_sharing_reuses_state_checkpoints(tmp_path):
    """Qwen3-Next-style hybrid with the unified radix cache: a later request that extends a finished
    one starts from the finished request's recurrent-state checkpoint and must produce exactly the
    tokens of a run without any sharing."""
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.parallel import state as ps
    cfg = dict(architectures=["Qwen3NextForCausalLM"], model_type="qwen3_next", hidden_size=64, intermediate_size=96,
               num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6,
               vocab_size=256, max_position_embeddings=512, full_attention_interval=2, linear_num_key_heads=2,
               linear_num_value_heads=4, linear_key_head_dim=8, linear_value_head_dim=8, linear_conv_kernel_dim=4,
               partial_rotary_factor=0.5, num_experts=0, tie_word_embeddings=False, torch_dtype="float32",
               layer_types=["linear_attention", "full_attention"] * 2)
    path = tmp_path / "q3n"
    path.mkdir()
    (path / "config.json").write_text(json.dumps(cfg))
    base = list(range(5, 45))
    sp = {"max_new_tokens": 6, "temperature": 0, "ignore_eos": True}

    def run(**kw):
        ps.reset_state()
        eng = Engine(model_path=str(path), device="cpu", dtype="float32", skip_tokenizer_init=True,
                     max_total_tokens=1024, enable_single_process=True, load_format="dummy",
                     **{"page_size": 1, **kw})
        try:
            first = eng.generate(input_ids=base, sampling_params=sp)
            cont = base + first["output_ids"][:5]                      # exactly the first request's cached tokens
            second = eng.generate(input_ids=cont + [77, 78, 79], sampling_params=sp)
            third = eng.generate(input_ids=[cont + [90, 91], base[:30] + [3, 3]], sampling_params=sp)
            tc = eng.scheduler.tree_cache
            if hasattr(tc, "assert_recurrent_slot_ledger"):
                tc.assert_recurrent_slot_ledger()
            eng.scheduler.check_memory()
            return (type(tc).__name__, first["output_ids"], second["output_ids"], [o["output_ids"] for o in third],
                    second["meta_info"]["cached_tokens"], [o["meta_info"]["cached_tokens"] for o in third],
                    getattr(tc, "snapshot_slots_in_use", lambda: 0)())
        finally:
            eng.shutdown()

    plain = run(disable_radix_cache=True)
    # overlap scheduling (the default): checkpoints come from the prefill steps only (here the end of the prompt)
    lapped = run()
    assert lapped[0] == "UnifiedRadixCache" and plain[0] == "ChunkCache"
    assert lapped[1:4] == plain[1:4] and lapped[4] == len(base) and lapped[5] == [len(base), 0]
    # sequential schedule: a finished request also checkpoints its final state
    shared = run(disable_overlap_schedule=True)
    assert shared[0] == "UnifiedRadixCache"
    assert shared[1:4] == plain[1:4]
    assert shared[4] == len(base) + 5                   # the second request started from the checkpoint
    assert shared[5][0] == len(base) + 5 and shared[5][1] == 0      # a prefix without a checkpoint is recomputed
    assert plain[4] == 0 and shared[6] >= 3
    # two snapshot slots only: checkpoints are recycled least-recently-used first and nothing leaks
    tight = run(recurrent_snapshot_slots=2, disable_overlap_schedule=True)
    assert tight[1:4] == plain[1:4] and tight[6] <= 2
    # pages of 4 tokens: the state is checkpointed at the last page boundary inside each prefill (here token 40 of
    # the first prompt), so later requests restart from there and still produce the unshared tokens
    paged = run(page_size=4)
    paged_plain = run(page_size=4, disable_radix_cache=True)
    assert paged[0] == "UnifiedRadixCache"
    assert paged[1:4] == paged_plain[1:4] == plain[1:4]
    assert paged[4] == 40 and paged[5] == [40, 0] and paged[6] >= 1
    # --max-recurrent-state-size counts request slots and checkpoint slots together
    sized = run(max_recurrent_state_size=264 + 3, disable_overlap_schedule=True)     # 256 + 8 request rows, 3 checkpoints
    assert sized[1:4] == plain[1:4] and sized[6] <= 3
    # with a host-memory KV tier the same tree logic runs over the host-tier radix tree
    hosted = run(hicache_storage="host", disable_overlap_schedule=True)
    assert hosted[0] == "UnifiedHiRadixCache"
    assert hosted[1:4] == plain[1:4] and hosted[4] == shared[4] and hosted[5] == shared[5]


@pytest.mark.parametrize("which", ["phi3", "mistral", "qwen2_moe", "deepseek_v2"])
def test_more_families_match_hf(tmp_path, which):
    """Phi-3 (fused qkv / gate_up checkpoint tensors), Mistral, Qwen2-MoE (biased attention, fused expert tensors,
    gated shared expert) and DeepSeek-V2 (MLA without a query LoRA, greedy routing)."""
    import transformers
    base = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, rms_norm_eps=1e-5, vocab_size=512, tie_word_embeddings=False,
                max_position_embeddings=512, rope_theta=10000.0)
    if which == "phi3":
        cfg = dict(base, pad_token_id=0, original_max_position_embeddings=512, partial_rotary_factor=1.0)
        hf, arch = transformers.Phi3ForCausalLM(transformers.Phi3Config(**cfg)), "Phi3ForCausalLM"
    elif which == "mistral":
        cfg = dict(base, sliding_window=None, head_dim=32)
        hf, arch = transformers.MistralForCausalLM(transformers.MistralConfig(**cfg)), "MistralForCausalLM"
    elif which == "qwen2_moe":
        cfg = dict(base, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                   shared_expert_intermediate_size=96, norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[],
                   use_sliding_window=False)
        hf, arch = transformers.Qwen2MoeForCausalLM(transformers.Qwen2MoeConfig(**cfg)), "Qwen2MoeForCausalLM"
    else:
        cfg = dict(base, num_hidden_layers=3, kv_lora_rank=32, q_lora_rank=None, qk_nope_head_dim=16,
                   qk_rope_head_dim=8, v_head_dim=16, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2,
                   moe_intermediate_size=64, first_k_dense_replace=1, routed_scaling_factor=1.0, topk_method="greedy",
                   n_group=1, topk_group=1, norm_topk_prob=False, num_key_value_heads=4)
        hf, arch = transformers.DeepseekV2ForCausalLM(transformers.DeepseekV2Config(**cfg)), "DeepseekV2ForCausalLM"
    hf = _init(hf)
    path = _save(str(tmp_path / which), hf, cfg, arch, which)
    assert _generate(path, PROMPTS, n=8) == _hf_generate(hf, PROMPTS, n=8)


@pytest.mark.parametrize("which", ["qwen2_vl", "qwen3_vl_moe"])
def test_vision_language_checkpoints_text_path_matches_hf(tmp_path, which):
    """Text-only prompts through the language half of Qwen2-VL and Qwen3-VL-MoE checkpoints (nested text config,
    weights under `model.language_model.`, vision tower present): three-stream rotary positions collapse to plain
    ones, and the expert count may be stored as `num_local_experts`."""
    import transformers
    if which == "qwen2_vl":
        text = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, rms_norm_eps=1e-6, vocab_size=512, max_position_embeddings=512,
                    rope_theta=10000.0, tie_word_embeddings=False,
                    rope_scaling={"type": "mrope", "mrope_section": [4, 6, 6]})
        vis = dict(depth=1, embed_dim=32, hidden_size=128, num_heads=2, patch_size=4, spatial_merge_size=2,
                   temporal_patch_size=2, in_channels=3, mlp_ratio=2)
        cfg = transformers.Qwen2VLConfig(text_config=text, vision_config=vis, image_token_id=500, video_token_id=501,
                                         vision_start_token_id=502, vision_end_token_id=503, tie_word_embeddings=False)
        hf, arch = transformers.Qwen2VLForConditionalGeneration(cfg), "Qwen2VLForConditionalGeneration"
    else:
        text = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6, vocab_size=512, max_position_embeddings=512,
                    rope_theta=10000.0, tie_word_embeddings=False, num_experts=8, num_experts_per_tok=2,
                    moe_intermediate_size=64, decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True,
                    rope_scaling={"rope_type": "default", "mrope_section": [4, 6, 6], "mrope_interleaved": True})
        vis = dict(depth=1, hidden_size=32, intermediate_size=64, num_heads=2, patch_size=4, spatial_merge_size=2,
                   temporal_patch_size=2, out_hidden_size=128, num_position_embeddings=64, deepstack_visual_indexes=[0],
                   in_channels=3)
        cfg = transformers.Qwen3VLMoeConfig(text_config=text, vision_config=vis, image_token_id=500,
                                            video_token_id=501, vision_start_token_id=502, vision_end_token_id=503,
                                            tie_word_embeddings=False)
        hf, arch = transformers.Qwen3VLMoeForConditionalGeneration(cfg), "Qwen3VLMoeForConditionalGeneration"
    hf = _init(hf)
    d = cfg.to_dict()
    d.pop("architectures", None)
    path = _save(str(tmp_path / which), hf, d, arch, which)
    assert _generate(path, PROMPTS, n=8) == _hf_generate(hf, PROMPTS, n=8)


def test_every_reference_architecture_name_resolves():
    """The `architectures[0]` strings the reference registers (`EntryClass` of each file under its `models/`)."""
    from sglang_jax_b200.models.registry import supported_architectures
    have = set(supported_architectures())
    ref = """BailingMoEForCausalLM BailingMoeForCausalLM BailingMoeV2ForCausalLM BailingMoeV2_5ForCausalLM
    DeepseekV3ForCausalLM DeepseekV2ForCausalLM DFlashDraftModel Gemma2ForCausalLM Gemma4ForCausalLM
    Gemma4ForConditionalGeneration Glm4MoeForCausalLM Glm5ForCausalLM GlmMoeDsaForCausalLM Grok1ForCausalLM
    KimiK25ForConditionalGeneration KimiLinearForCausalLM LlamaForCausalLM Phi3ForCausalLM InternLM3ForCausalLM
    LlamaForCausalLMEagle3 MiMoForCausalLM MiMoMTPForCausalLM MiMoV2FlashForCausalLM MiMoV2MTPForCausalLM
    MiMoV2ForCausalLM MiniMaxM2ForCausalLM QWenLMHeadModel Qwen2ForCausalLM Qwen2MoeForCausalLM Qwen3ForCausalLM
    Qwen3_5MoeForConditionalGeneration Qwen3_5ForConditionalGeneration Qwen3MoeForCausalLM UMT5EncoderModel
    UMT5DecoderModel UMT5Model UMT5ForConditionalGeneration""".split()
    assert [r for r in ref if r not in have] == []
