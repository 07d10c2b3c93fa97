"""LoRA serving on CPU: an adapter applied through the stacked-buffer path equals the same
model with the low-rank update merged into its weights; adapters can be mixed in one batch,
loaded and unloaded at run time (reference tests: `python/sgl_jax/test/lora/`)."""

import json
import os

import pytest
import torch

from sglang_jax_b200.utils.tiny_models import TINY_QWEN3, tiny_qwen3_state_dict, write_config_only


def _write_adapter(path, seed, r=8, alpha=16.0, targets=("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"),
                   cfg=TINY_QWEN3, scale=0.05):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    dims = {"q_proj": (H, nh * D), "k_proj": (H, nkv * D), "v_proj": (H, nkv * D), "o_proj": (nh * D, H),
            "gate_proj": (H, I), "up_proj": (H, I), "down_proj": (I, H)}
    sd = {}
    for i in range(cfg["num_hidden_layers"]):
        for m in targets:
            fin, fout = dims[m]
            blk = "self_attn" if m in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
            p = f"base_model.model.model.layers.{i}.{blk}.{m}."
            sd[p + "lora_A.weight"] = torch.empty(r, fin).normal_(0, scale, generator=g)
            sd[p + "lora_B.weight"] = torch.empty(fout, r).normal_(0, scale, generator=g)
    save_file(sd, os.path.join(path, "adapter_model.safetensors"))
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump({"r": r, "lora_alpha": alpha, "target_modules": list(targets), "peft_type": "LORA"}, f)
    return sd, alpha / r


def _write_merged(path, base_sd, adapter_sd, scaling):
    from safetensors.torch import save_file
    sd = {k: v.clone() for k, v in base_sd.items()}
    for k, a in adapter_sd.items():
        if "lora_A" not in k:
            continue
        b = adapter_sd[k.replace("lora_A", "lora_B")]
        name = k.replace("base_model.model.", "").replace(".lora_A.weight", ".weight")
        sd[name] = sd[name] + scaling * (b @ a)
    write_config_only(path, TINY_QWEN3)
    save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(path, "model.safetensors"))
    return path


@pytest.fixture(scope="module")
def env(tmp_path_factory):
    from safetensors.torch import save_file
    root = tmp_path_factory.mktemp("lora")
    base_sd = tiny_qwen3_state_dict(TINY_QWEN3, 0)
    base = write_config_only(str(root / "base"), TINY_QWEN3)
    save_file({k: v.contiguous() for k, v in base_sd.items()}, os.path.join(base, "model.safetensors"))
    out = {"base": base, "base_sd": base_sd}
    for name, seed, r in (("a", 11, 8), ("b", 12, 4)):
        sd, sc = _write_adapter(str(root / name), seed, r=r)
        out[name] = str(root / name)
        out[name + "_merged"] = _write_merged(str(root / (name + "_merged")), base_sd, sd, sc)
    return out


PROMPTS = [[3, 17, 42, 9, 5, 11, 8], [4, 4, 19, 23, 77, 12], [9, 8, 7, 6, 5, 4, 3, 2]]
SP = {"temperature": 0.0, "max_new_tokens": 10, "ignore_eos": True}


def _run(model_path, prompts, lora_path=None, **kw):
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.parallel import state as ps
    ps.reset_state()
    eng = Engine(model_path=model_path, device="cpu", enable_single_process=True, page_size=4,
                 skip_tokenizer_init=True, max_total_tokens=2048, dtype="float32", log_level="error", **kw)
    try:
        outs = eng.generate(input_ids=prompts, sampling_params=SP, lora_path=lora_path)
        return [o["output_ids"] for o in outs], eng
    finally:
        eng.shutdown()


def test_adapter_equals_merged_weights_and_mixed_batch(env):
    want_a, _ = _run(env["a_merged"], PROMPTS)
    want_b, _ = _run(env["b_merged"], PROMPTS)
    want_base, _ = _run(env["base"], PROMPTS)
    assert want_a != want_base and want_b != want_base
    kw = dict(lora_paths=[f"a={env['a']}", f"b={env['b']}"], max_loras_per_batch=2)
    got_a, _ = _run(env["base"], PROMPTS, lora_path=["a"] * 3, **kw)
    assert got_a == want_a
    # one batch mixing both adapters and the base model
    mixed, _ = _run(env["base"], PROMPTS, lora_path=["a", "b", None], **kw)
    assert mixed == [want_a[0], want_b[1], want_base[2]]


def test_static_lora_applies_the_first_adapter_to_every_request(env):
    """`--enable-static-lora`: requests need not name an adapter; the first loaded one serves them all."""
    want_a, _ = _run(env["a_merged"], PROMPTS)
    got, _ = _run(env["base"], PROMPTS, lora_path=None, lora_paths=[f"a={env['a']}", f"b={env['b']}"],
                  max_loras_per_batch=2, enable_static_lora=True)
    assert got == want_a
    got, _ = _run(env["base"], PROMPTS, lora_path=["b", None, "b"], lora_paths=[f"a={env['a']}", f"b={env['b']}"],
                  max_loras_per_batch=2, enable_static_lora=True)
    assert got == want_a


def test_more_adapters_than_slots_are_served_in_turns(env):
    want_a, _ = _run(env["a_merged"], PROMPTS[:1])
    want_b, _ = _run(env["b_merged"], PROMPTS[1:2])
    got, _ = _run(env["base"], PROMPTS[:2], lora_path=["a", "b"], lora_paths=[f"a={env['a']}", f"b={env['b']}"],
                  max_loras_per_batch=1, max_loaded_loras=2)
    assert got == [want_a[0], want_b[0]]


def test_dynamic_load_and_unload(env):
    from sglang_jax_b200.entrypoints.engine import Engine
    from sglang_jax_b200.parallel import state as ps
    ps.reset_state()
    eng = Engine(model_path=env["base"], device="cpu", enable_single_process=True, page_size=4,
                 skip_tokenizer_init=True, max_total_tokens=2048, dtype="float32", log_level="error",
                 enable_lora=True, max_lora_rank=8, lora_target_modules=["all"], max_loras_per_batch=2)
    try:
        with pytest.raises(Exception):
            eng.generate(input_ids=PROMPTS[:1], sampling_params=SP, lora_path=["a"])
        res = eng.load_lora_adapter("a", env["a"])
        assert res.success and res.loaded_adapters == {"a": env["a"]}
        assert not eng.load_lora_adapter("a", env["a"]).success
        got = eng.generate(input_ids=PROMPTS[:1], sampling_params=SP, lora_path=["a"])[0]["output_ids"]
        res = eng.unload_lora_adapter("a")
        assert res.success and res.loaded_adapters == {}
        with pytest.raises(Exception):
            eng.generate(input_ids=PROMPTS[:1], sampling_params=SP, lora_path=["a"])
        assert not eng.unload_lora_adapter("a").success
    finally:
        eng.shutdown()
    want, _ = _run(env["a_merged"], PROMPTS[:1])
    assert got == want[0]


def test_registry_counts_in_flight():
    import asyncio
    from sglang_jax_b200.lora.lora_registry import LoRARegistry
    reg = LoRARegistry(["x=/p/x", {"lora_name": "y", "lora_path": "/p/y", "pinned": True}])
    ix = reg.acquire("x")
    assert reg.in_flight(ix) == 1 and reg.acquire(["x", "y"])[0] == ix and reg.in_flight(ix) == 2
    with pytest.raises(ValueError):
        reg.acquire("zzz")

    async def go():
        lid = reg.unregister("x")
        waiter = asyncio.create_task(reg.wait_for_unload(lid))
        await asyncio.sleep(0.01)
        assert not waiter.done()
        reg.release(lid)
        reg.release(lid)
        await asyncio.wait_for(waiter, 1)

    asyncio.run(go())
    assert reg.get("x") is None and reg.get("y").pinned
