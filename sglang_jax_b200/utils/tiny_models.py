"""Synthetic checkpoints in HF layout, for tests, the plumbing oracle and benchmarks.

`write_tiny_qwen3_checkpoint` produces the tiny Qwen3-style decoder of the CPU plumbing
config: 2 layers, hidden 256, 4 query / 2 KV heads, head_dim 64 with per-head q/k RMSNorm,
SwiGLU FFN 512, RMSNorm eps 1e-6, RoPE theta 1e6, vocab 1024, tied embeddings, weights
normal(0, 0.02) from seed 0.  The reference's own `dummy` load format writes zeros
(`python/sgl_jax/srt/utils/weight_utils.py:2360`), hence a real checkpoint.
"""

from __future__ import annotations

import json
import os

import torch

TINY_QWEN3 = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=256, intermediate_size=512,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6,
    rope_theta=1000000.0, vocab_size=1024, tie_word_embeddings=True, max_position_embeddings=4096,
    hidden_act="silu", attention_bias=False, torch_dtype="float32", bos_token_id=None, eos_token_id=None,
)

ARCH_CONFIGS = {
    "llama3-8b": dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=4096,
                      intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0,
                      vocab_size=128256, tie_word_embeddings=False, max_position_embeddings=8192,
                      torch_dtype="bfloat16"),
    "qwen3-32b": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=5120,
                      intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                      num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                      vocab_size=151936, tie_word_embeddings=False, max_position_embeddings=40960,
                      torch_dtype="bfloat16"),
    # the per-rank shard of Qwen3-32B under 8-way tensor parallelism as a model of its own (8 query heads, 1 KV head,
    # intermediate 3200, vocabulary 18992): run on ONE GPU it shows what a rank computes when communication is free
    "qwen3-32b-tp8-shard": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=5120,
                                intermediate_size=3200, num_hidden_layers=64, num_attention_heads=8,
                                num_key_value_heads=1, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                                vocab_size=18992, tie_word_embeddings=False, max_position_embeddings=40960,
                                torch_dtype="bfloat16"),
    "qwen3-8b": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096,
                     intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                     num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                     vocab_size=151936, tie_word_embeddings=False, max_position_embeddings=40960,
                     torch_dtype="bfloat16"),
    "qwen3-30b-a3b": dict(architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", hidden_size=2048,
                          intermediate_size=6144, moe_intermediate_size=768, num_hidden_layers=48,
                          num_attention_heads=32, num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6,
                          rope_theta=1000000.0, vocab_size=151936, num_experts=128, num_experts_per_tok=8,
                          norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[],
                          tie_word_embeddings=False, max_position_embeddings=40960, torch_dtype="bfloat16"),
    "deepseek-v3": dict(architectures=["DeepseekV3ForCausalLM"], model_type="deepseek_v3", hidden_size=7168,
                        intermediate_size=18432, moe_intermediate_size=2048, num_hidden_layers=61,
                        num_attention_heads=128, num_key_value_heads=128, q_lora_rank=1536, kv_lora_rank=512,
                        qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, n_routed_experts=256,
                        n_shared_experts=1, num_experts_per_tok=8, n_group=8, topk_group=4,
                        scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True,
                        routed_scaling_factor=2.5, first_k_dense_replace=3, moe_layer_freq=1,
                        rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=129280, tie_word_embeddings=False,
                        max_position_embeddings=163840, torch_dtype="bfloat16",
                        rope_scaling=dict(type="yarn", factor=40, original_max_position_embeddings=4096,
                                          beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0)),
}


def write_config_only(path: str, config: dict) -> str:
    """A model directory with only `config.json`: enough for `--load-format dummy`."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    return path


def tiny_qwen3_state_dict(config: dict = TINY_QWEN3, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    H, I, V = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    nh, nkv, D = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]

    def w(*shape):
        return torch.empty(*shape, dtype=torch.float32).normal_(0, std, generator=g)

    sd = {"model.embed_tokens.weight": w(V, H)}
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}."
        sd[p + "self_attn.q_proj.weight"] = w(nh * D, H)
        sd[p + "self_attn.k_proj.weight"] = w(nkv * D, H)
        sd[p + "self_attn.v_proj.weight"] = w(nkv * D, H)
        sd[p + "self_attn.o_proj.weight"] = w(H, nh * D)
        if config.get("attention_bias"):
            sd[p + "self_attn.q_proj.bias"] = w(nh * D)
            sd[p + "self_attn.k_proj.bias"] = w(nkv * D)
            sd[p + "self_attn.v_proj.bias"] = w(nkv * D)
            sd[p + "self_attn.o_proj.bias"] = w(H)
        sd[p + "self_attn.q_norm.weight"] = torch.ones(D)
        sd[p + "self_attn.k_norm.weight"] = torch.ones(D)
        sd[p + "mlp.gate_proj.weight"] = w(I, H)
        sd[p + "mlp.up_proj.weight"] = w(I, H)
        sd[p + "mlp.down_proj.weight"] = w(H, I)
        sd[p + "input_layernorm.weight"] = torch.ones(H)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(H)
    sd["model.norm.weight"] = torch.ones(H)
    if not config.get("tie_word_embeddings", False):
        sd["lm_head.weight"] = w(V, H)
    return sd


def write_tiny_qwen3_checkpoint(path: str, seed: int = 0, config: dict | None = None, dtype=torch.float32,
                                std: float = 0.02) -> str:
    from safetensors.torch import save_file
    cfg = dict(config or TINY_QWEN3)
    write_config_only(path, cfg)
    sd = {k: v.to(dtype).contiguous() for k, v in tiny_qwen3_state_dict(cfg, seed, std).items()}
    if cfg.get("model_type") == "llama":
        sd = {k: v for k, v in sd.items() if "q_norm" not in k and "k_norm" not in k}
    save_file(sd, os.path.join(path, "model.safetensors"))
    return path


def write_tiny_eagle_checkpoint(path: str, target_config: dict = TINY_QWEN3, kind: str = "eagle", seed: int = 3,
                                draft_vocab_size: int | None = None) -> str:
    """A random EAGLE (`kind="eagle"`) or EAGLE-3 (`kind="eagle3"`) draft head sized for
    `target_config`, in the layout those checkpoints use (no embedding table; EAGLE shares
    the target LM head, EAGLE-3 has its own, optionally over a reduced vocabulary)."""
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)
    H, I, V = target_config["hidden_size"], target_config["intermediate_size"], target_config["vocab_size"]
    nh, nkv, D = target_config["num_attention_heads"], target_config["num_key_value_heads"], target_config["head_dim"]

    def w(*shape):
        return torch.empty(*shape, dtype=torch.float32).normal_(0, 0.02, generator=g)

    cfg = dict(target_config)
    cfg["num_hidden_layers"] = 1
    cfg["model_type"] = "llama"
    cfg["tie_word_embeddings"] = False
    sd = {}
    if kind == "eagle":
        cfg["architectures"] = ["LlamaForCausalLMEagle"]
        pre = "layers.0."
        qkv_in = H
        sd["fc.weight"] = w(H, 2 * H)
        sd["fc.bias"] = torch.zeros(H)
    else:
        cfg["architectures"] = ["LlamaForCausalLMEagle3"]
        dv = draft_vocab_size or V
        cfg["draft_vocab_size"] = dv
        pre = "midlayer."
        qkv_in = 2 * H
        sd["fc.weight"] = w(H, 3 * H)
        sd[pre + "input_layernorm.weight"] = torch.ones(H)
        sd[pre + "hidden_norm.weight"] = torch.ones(H)
        sd["norm.weight"] = torch.ones(H)
        sd["lm_head.weight"] = w(dv, H)
        if dv != V:
            # draft id i stands for target id i * (V // dv)
            sd["d2t"] = (torch.arange(dv) * (V // dv) - torch.arange(dv)).to(torch.int64)
    sd[pre + "self_attn.q_proj.weight"] = w(nh * D, qkv_in)
    sd[pre + "self_attn.k_proj.weight"] = w(nkv * D, qkv_in)
    sd[pre + "self_attn.v_proj.weight"] = w(nkv * D, qkv_in)
    sd[pre + "self_attn.o_proj.weight"] = w(H, nh * D)
    sd[pre + "mlp.gate_proj.weight"] = w(I, H)
    sd[pre + "mlp.up_proj.weight"] = w(I, H)
    sd[pre + "mlp.down_proj.weight"] = w(H, I)
    sd[pre + "post_attention_layernorm.weight"] = torch.ones(H)
    write_config_only(path, cfg)
    save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(path, "model.safetensors"))
    return path


def write_tiny_mimo_checkpoint(path: str, seed: int = 0, num_mtp_layers: int = 1) -> str:
    """A tiny MiMo-style checkpoint: Qwen2 decoder (biased q/k/v) plus `model.mtp_layers.*`."""
    from safetensors.torch import save_file
    cfg = dict(TINY_QWEN3, architectures=["MiMoForCausalLM"], model_type="mimo", tie_word_embeddings=False,
               num_nextn_predict_layers=num_mtp_layers)
    g = torch.Generator().manual_seed(seed + 100)
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def w(*shape):
        return torch.empty(*shape, dtype=torch.float32).normal_(0, 0.02, generator=g)

    sd = {k: v for k, v in tiny_qwen3_state_dict(cfg, seed).items() if "q_norm" not in k and "k_norm" not in k}
    prefixes = [f"model.layers.{i}." for i in range(cfg["num_hidden_layers"])] + \
        [f"model.mtp_layers.{j}." for j in range(num_mtp_layers)]
    for p in prefixes:
        sd[p + "self_attn.q_proj.bias"] = w(nh * D)
        sd[p + "self_attn.k_proj.bias"] = w(nkv * D)
        sd[p + "self_attn.v_proj.bias"] = w(nkv * D)
    for j in range(num_mtp_layers):
        p = f"model.mtp_layers.{j}."
        sd[p + "token_layernorm.weight"] = torch.ones(H)
        sd[p + "hidden_layernorm.weight"] = torch.ones(H)
        sd[p + "input_proj.weight"] = w(H, 2 * H)
        sd[p + "input_layernorm.weight"] = torch.ones(H)
        sd[p + "self_attn.q_proj.weight"] = w(nh * D, H)
        sd[p + "self_attn.k_proj.weight"] = w(nkv * D, H)
        sd[p + "self_attn.v_proj.weight"] = w(nkv * D, H)
        sd[p + "self_attn.o_proj.weight"] = w(H, nh * D)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(H)
        sd[p + "mlp.gate_proj.weight"] = w(I, H)
        sd[p + "mlp.up_proj.weight"] = w(I, H)
        sd[p + "mlp.down_proj.weight"] = w(H, I)
        sd[p + "final_layernorm.weight"] = torch.ones(H)
    write_config_only(path, cfg)
    save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(path, "model.safetensors"))
    return path


def write_tiny_dflash_checkpoint(path: str, target_config: dict = TINY_QWEN3, seed: int = 5, block_size: int = 4,
                                 target_layer_ids=(0, 1)) -> str:
    """A random DFlash block drafter (one Qwen3-style layer, no embedding / head)."""
    from safetensors.torch import save_file
    cfg = dict(target_config, architectures=["DFlashDraftModel"], num_hidden_layers=1, tie_word_embeddings=False,
               dflash_config=dict(target_layer_ids=list(target_layer_ids), block_size=block_size,
                                  mask_token_id=target_config["vocab_size"] - 1))
    sd = {k[len("model."):]: v for k, v in tiny_qwen3_state_dict(dict(cfg, tie_word_embeddings=True), seed).items()
          if k.startswith("model.layers.") or k == "model.norm.weight"}
    g = torch.Generator().manual_seed(seed)
    H = cfg["hidden_size"]
    sd["fc.weight"] = torch.empty(H, len(target_layer_ids) * H).normal_(0, 0.02, generator=g)
    sd["hidden_norm.weight"] = torch.ones(H)
    write_config_only(path, cfg)
    save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(path, "model.safetensors"))
    return path
