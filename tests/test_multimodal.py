"""Multimodal pipeline on CPU: encoder / ViT parity with HF, solver behaviour, and whole
pipelines (text -> DiT -> VAE, image -> ViT -> LLM) through the global scheduler and the HTTP
layer (reference tests: `python/sgl_jax/test/multimodal/`)."""

import base64
import io
import json
import os
import threading
import time

import numpy as np
import pytest
import torch


def test_qwen2_5_vl_vision_transformer_matches_hf():
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLVisionConfig
    from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VisionTransformerPretrainedModel
    from sglang_jax_b200.multimodal.models.qwen2_5_vl_vit import Qwen2_5_VisionTransformer
    cfg = Qwen2_5_VLVisionConfig(depth=4, hidden_size=64, intermediate_size=96, num_heads=4, in_channels=3,
                                 patch_size=4, spatial_merge_size=2, temporal_patch_size=2, window_size=16,
                                 fullatt_block_indexes=[1, 3], out_hidden_size=48)
    torch.manual_seed(0)
    hf = Qwen2_5_VisionTransformerPretrainedModel._from_config(cfg, attn_implementation="sdpa").float().eval()
    for p in hf.parameters():
        p.data.normal_(0, 0.08) if p.dim() > 1 else p.data.uniform_(0.5, 1.5)
    mine = Qwen2_5_VisionTransformer(cfg, dtype=torch.float32)
    loaded = mine.load_weights(hf.state_dict().items())
    assert loaded == {n for n, _ in mine.named_parameters()}, set(dict(mine.named_parameters())) - loaded
    grid = torch.tensor([[1, 6, 10], [1, 4, 4]])
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(n, 3 * 2 * 4 * 4)
    with torch.no_grad():
        want = hf(px, grid_thw=grid).pooler_output
    got = mine(px, grid)
    assert got.shape == want.shape == (n // 4, 48)
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()


def test_flow_solvers_converge_on_a_known_velocity_field():
    """With the exact velocity of a point mass at `x0` (v = (x - x0) / sigma) every flow solver must
    land on x0, whatever the number of steps; the second-order solver is exact for this field too."""
    from sglang_jax_b200.multimodal.models.diffusion_solvers import (FlowMatchEulerDiscreteScheduler,
                                                                       UniPCMultistepScheduler, shifted_sigmas)
    s = shifted_sigmas(8, 3.0)
    assert s[0] == 1 and s[-1] == 0 and bool((s[:-1] > s[1:]).all())
    x0 = torch.tensor([[1.5, -2.0, 0.25]])
    for cls in (FlowMatchEulerDiscreteScheduler, UniPCMultistepScheduler):
        for steps in (4, 16):
            sch = cls(shift=3.0)
            sch.set_timesteps(steps)
            x = torch.randn(1, 3, generator=torch.Generator().manual_seed(1))
            for i in range(steps):
                sigma = sch.sigmas[i]
                x = sch.step((x - x0) / sigma, x)
            assert torch.allclose(x, x0, atol=1e-4), (cls.__name__, steps, x)
    # a curved field: the multistep solver beats Euler at equal cost
    def run(cls, steps):
        sch = cls(shift=1.0)
        sch.set_timesteps(steps)
        x = torch.ones(1, 1) * 2.0
        for i in range(steps):
            sg = sch.sigmas[i]
            x0_hat = torch.tanh(x) * (1 - sg) + 0.3            # a smooth, sigma-dependent denoiser
            x = sch.step((x - x0_hat) / sg, x)
        return x
    ref = run(FlowMatchEulerDiscreteScheduler, 2000)
    e_euler = (run(FlowMatchEulerDiscreteScheduler, 10) - ref).abs().item()
    e_unipc = (run(UniPCMultistepScheduler, 10) - ref).abs().item()
    assert e_unipc < e_euler, (e_unipc, e_euler)


T5 = dict(vocab_size=259, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_heads=4, relative_attention_num_buckets=32,
          relative_attention_max_distance=128, layer_norm_epsilon=1e-6, is_gated_act=True, dense_act_fn="gelu_new")
DIT = dict(in_channels=4, out_channels=4, patch_size=[1, 2, 2], num_attention_heads=2, attention_head_dim=24,
           ffn_dim=96, num_layers=2, text_dim=32, freq_dim=32)
VAE = dict(z_dim=4, base_dim=8, dim_mult=[4, 2, 1, 1], temporal_upsample=[True, True, False], out_channels=3,
           scaling_factor=1.0)


@pytest.fixture(scope="module")
def wan_server():
    from sglang_jax_b200.multimodal.entrypoint.http_server import MultimodalServer
    srv = MultimodalServer("Wan-AI/Wan2.1-T2V-1.3B-Diffusers", None, config_overrides={0: T5, 1: DIT, 2: VAE})
    yield srv
    srv.shutdown()


def test_text_to_video_pipeline_over_http(wan_server):
    from fastapi.testclient import TestClient
    from sglang_jax_b200.multimodal.entrypoint.http_server import build_app
    with TestClient(build_app(wan_server)) as c:
        h = c.get("/health").json()
        assert [s["scheduler"] for s in h["stages"]] == ["text_encoder", "diffusion", "vae"]
        body = {"prompt": "a red fox", "negative_prompt": "blurry", "size": "32x32", "num_frames": 5,
                "num_inference_steps": 3, "guidance_scale": 3.0, "seed": 7}
        r = c.post("/api/v1/videos/generation", json=body)
        assert r.status_code == 200, r.text
        d = r.json()["data"]
        assert d["width"] == 32 and d["height"] == 32 and d["num_frames"] == 5
        png = base64.b64decode(d["b64_png"][0])
        assert png[:8] == bytes([0x89, 0x50, 0x4E, 0x47, 0x0D, 0x0A, 0x1A, 0x0A])
        again = c.post("/api/v1/videos/generation", json=body).json()["data"]
        assert again["b64_png"] == d["b64_png"]                          # seeded: bit-identical
        other = c.post("/api/v1/videos/generation", json=dict(body, seed=8)).json()["data"]
        assert other["b64_png"] != d["b64_png"]
        img = c.post("/api/v1/images/generation", json={"prompt": "x", "size": "16x16", "num_inference_steps": 2})
        assert img.status_code == 200 and img.json()["data"]["num_frames"] == 1
        assert c.post("/v1/chat/completions", json={"input_ids": [1]}).status_code == 400     # no llm stage here
        assert set(r.json()["meta"]["stage_times"]) == {"0", "1", "2"}


def test_abort_reaches_the_stage_holding_the_request(wan_server):
    from sglang_jax_b200.multimodal.manager.io_struct import GenerateMMReqInput
    import asyncio
    gs = wan_server.gs
    diff = gs.stages[1].scheduler
    orig = diff.model.forward
    started = threading.Event()

    def slow(*a, **k):
        started.set()
        time.sleep(0.05)
        return orig(*a, **k)

    diff.model.forward = slow
    try:
        async def go():
            obj = GenerateMMReqInput(prompt="p", height=16, width=16, num_inference_steps=200, rid="abort-me")
            task = asyncio.create_task(wan_server.tok.generate(obj))
            while not started.is_set():
                await asyncio.sleep(0.01)
            assert gs.abort("abort-me")
            return await asyncio.wait_for(task, 20)
        before = diff.steps_run
        out = asyncio.run(go())
        assert out.error == "aborted" and diff.steps_run - before < 200
        assert not gs.abort("abort-me")
    finally:
        diff.model.forward = orig


def test_vision_language_pipeline(tmp_path):
    """image patches -> ViT stage -> embeddings spliced over placeholder tokens -> LLM stage; the
    answer must equal running the language model alone on the same spliced embeddings."""
    from fastapi.testclient import TestClient
    from sglang_jax_b200.multimodal.entrypoint.http_server import MultimodalServer, build_app
    from sglang_jax_b200.utils.tiny_models import TINY_QWEN3, write_tiny_qwen3_checkpoint
    llm = write_tiny_qwen3_checkpoint(str(tmp_path / "llm"), config=dict(TINY_QWEN3, tie_word_embeddings=False))
    vit = dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4,
               spatial_merge_size=2, temporal_patch_size=2, window_size=16, fullatt_block_indexes=[1],
               out_hidden_size=TINY_QWEN3["hidden_size"])
    srv = MultimodalServer("Qwen/Qwen2.5-VL-7B-Instruct", None,
                           config_overrides={0: vit, 1: {"model_path": llm, "image_token_id": 900}})
    try:
        grid = [[1, 4, 4]]
        px = torch.randn(16, 3 * 2 * 4 * 4, generator=torch.Generator().manual_seed(3))
        ids = [5, 6] + [900] * 4 + [7, 8, 9]
        with TestClient(build_app(srv)) as c:
            r = c.post("/v1/chat/completions", json={"input_ids": ids, "pixel_values": px.tolist(),
                                                     "image_grid_thw": grid, "max_tokens": 6})
            assert r.status_code == 200, r.text
            got = r.json()["choices"][0]["message"]["output_ids"]
            bad = c.post("/v1/chat/completions", json={"input_ids": [5, 900, 7], "pixel_values": px.tolist(),
                                                       "image_grid_thw": grid})
            assert bad.status_code == 500 and "placeholder" in bad.json()["error"]["message"]
        vit_model = srv.gs.stages[0].scheduler.model
        llm_stage = srv.gs.stages[1].scheduler
        emb = vit_model(px, torch.tensor(grid))
        table = llm_stage.runner.model.get_embed_and_head()[0]
        x = table[torch.tensor(ids)].clone()
        x[2:6] = emb
        want = llm_stage.gen.generate(ids, x, 6)
        assert got == want and len(got) == 6
        text_only = llm_stage.gen.generate(ids, None, 6)
        assert text_only != got                               # the image really conditions the answer
    finally:
        srv.shutdown()


def test_speech_pipeline_roundtrip(tmp_path):
    from fastapi.testclient import TestClient
    from sglang_jax_b200.multimodal.entrypoint.http_server import MultimodalServer, build_app
    from sglang_jax_b200.utils.tiny_models import TINY_QWEN3, write_tiny_qwen3_checkpoint
    llm = write_tiny_qwen3_checkpoint(str(tmp_path / "llm"))
    codec = dict(sample_rate=8000, n_mels=20, d_model=32, heads=2, layers=1, num_quantizers=2, codebook_size=64, hop=80)
    srv = MultimodalServer("XiaomiMiMo/MiMo-Audio", None, config_overrides={
        0: codec, 1: {"model_path": llm, "audio_token_offset": 300, "codebook_size": 64, "num_quantizers": 2}, 2: codec})
    try:
        with TestClient(build_app(srv)) as c:
            wave = np.sin(np.linspace(0, 200, 4000)).astype("<f4")
            asr = c.post("/v1/audio/transcriptions", json={"audio_b64": base64.b64encode(wave.tobytes()).decode(),
                                                           "max_new_tokens": 5})
            assert asr.status_code == 200 and len(asr.json()["output_ids"]) == 5
            tts = c.post("/v1/audio/speech", json={"input": "hello", "max_new_tokens": 6})
            assert tts.status_code == 200 and tts.content[:4] == b"RIFF" and len(tts.content) > 44 + 100
        tok = srv.gs.stages[0].scheduler.model
        codes = tok.encode(torch.from_numpy(wave.copy()))
        assert codes.shape[1] == 2 and int(codes.max()) < 64
        assert torch.equal(codes, tok.encode(torch.from_numpy(wave.copy())))
    finally:
        srv.shutdown()


def test_clip_text_and_vision_towers_match_hf():
    from transformers import CLIPTextConfig, CLIPTextModel as HFText, CLIPVisionConfig, CLIPVisionModel as HFVision
    from sglang_jax_b200.multimodal.models.clip import CLIPTextModel, CLIPVisionModel
    torch.manual_seed(0)
    tc = CLIPTextConfig(vocab_size=120, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                        num_attention_heads=4, max_position_embeddings=32, eos_token_id=2, bos_token_id=1)
    hf = HFText(tc).float().eval()
    mine = CLIPTextModel(tc, dtype=torch.float32)
    loaded = mine.load_weights(hf.state_dict().items())
    assert loaded == {n for n, _ in mine.named_parameters()}
    ids = torch.randint(3, 119, (2, 17))
    ids[0, 9] = 119
    ids[1, 16] = 119                      # the end-of-text token carries the largest id
    with torch.no_grad():
        want = hf(input_ids=ids)
        got, pooled = mine(ids, return_pooled=True)
    assert torch.allclose(got, want.last_hidden_state, atol=2e-5)
    assert torch.allclose(pooled, want.pooler_output, atol=2e-5)
    vc = CLIPVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                          image_size=32, patch_size=8)
    hfv = HFVision(vc).float().eval()
    mv = CLIPVisionModel(vc, dtype=torch.float32)
    loaded = mv.load_weights(hfv.state_dict().items())
    assert loaded == {n for n, _ in mv.named_parameters()}
    px = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        want = hfv(pixel_values=px)
        got, pooled = mv(px, return_pooled=True)
    assert torch.allclose(got, want.last_hidden_state, atol=2e-5)
    assert torch.allclose(pooled, want.pooler_output, atol=2e-5)


FLUX = dict(in_channels=16, num_layers=2, num_single_layers=2, attention_head_dim=16, num_attention_heads=2,
            joint_attention_dim=32, pooled_projection_dim=24, guidance_embeds=True, axes_dims_rope=[4, 6, 6])


def test_flux_dit_structure():
    from types import SimpleNamespace
    from sglang_jax_b200.multimodal.model_executor.loading import init_dummy
    from sglang_jax_b200.multimodal.models.flux import FluxTransformer2DModel, rope_nd
    m = init_dummy(FluxTransformer2DModel(SimpleNamespace(**FLUX), dtype=torch.float32), seed=3, std=0.05).eval()
    names = {n for n, _ in m.named_parameters()}
    for n in ("x_embedder.weight", "context_embedder.bias", "time_text_embed.guidance_embedder.linear_2.weight",
              "time_text_embed.text_embedder.linear_1.weight", "transformer_blocks.1.norm1_context.linear.weight",
              "transformer_blocks.0.attn.norm_added_k.weight", "transformer_blocks.0.attn.to_add_out.bias",
              "transformer_blocks.0.ff_context.net.0.proj.weight", "transformer_blocks.0.ff.net.2.bias",
              "single_transformer_blocks.1.proj_mlp.weight", "single_transformer_blocks.0.attn.norm_q.weight",
              "single_transformer_blocks.0.proj_out.weight", "norm_out.linear.weight", "proj_out.bias"):
        assert n in names, n                                       # the published checkpoint's tensor names
    assert m.single_transformer_blocks[0].proj_out.weight.shape == (32, 5 * 32)
    g = torch.Generator().manual_seed(0)
    lat = torch.randn(2, 4, 1, 8, 12, generator=g)
    text = torch.randn(2, 5, 32, generator=g)
    pooled = torch.randn(2, 24, generator=g)
    t = torch.tensor([500.0, 20.0])
    v = m(lat, t, text, pooled, torch.tensor([3.5, 1.0]))
    assert v.shape == lat.shape and torch.isfinite(v).all()
    # batch rows are independent and each conditioning input matters
    v0 = m(lat[:1], t[:1], text[:1], pooled[:1], torch.tensor([3.5]))
    assert torch.allclose(v0, v[:1], atol=1e-5)
    assert not torch.allclose(m(lat[:1], t[:1], text[:1], pooled[1:], torch.tensor([3.5])), v0, atol=1e-4)
    assert not torch.allclose(m(lat[:1], t[:1], text[:1], pooled[:1], torch.tensor([1.0])), v0, atol=1e-4)
    assert not torch.allclose(m(lat[:1], t[:1], text[1:], pooled[:1], torch.tensor([3.5])), v0, atol=1e-4)
    # text tokens sit at the rotary origin: their order only matters through the text weights, so
    # permuting them permutes nothing in the image output
    perm = torch.tensor([3, 0, 4, 1, 2])
    assert torch.allclose(m(lat[:1], t[:1], text[:1, perm], pooled[:1], torch.tensor([3.5])), v0, atol=1e-5)
    # zero output gates (adaLN-zero at initialisation) make every block the identity
    saved = {}
    for n, p in m.named_parameters():
        if n.endswith("norm1.linear.weight") or n.endswith("norm1.linear.bias") or ".norm.linear." in n:
            saved[n] = p.data.clone()
            p.data.zero_()
    x_only = m(lat[:1], t[:1], text[:1], pooled[:1], torch.tensor([3.5]))
    other_text = m(lat[:1], t[:1], text[1:], pooled[:1], torch.tensor([3.5]))
    assert torch.allclose(x_only, other_text, atol=1e-6)           # the image stream never saw the text
    cos, sin = rope_nd(torch.tensor([[0., 0., 0.], [0., 2., 5.]]), (4, 6, 6))
    assert cos.shape == (2, 8) and torch.allclose(cos[0], torch.ones(8)) and torch.allclose(sin[0], torch.zeros(8))
    assert torch.allclose(cos[1, :2], torch.ones(2))               # first band follows axis 0, which is 0 here


def test_flux_text_to_image_pipeline_with_pooled_clip_prompt(tmp_path):
    import json
    from fastapi.testclient import TestClient
    from sglang_jax_b200.multimodal.entrypoint.http_server import MultimodalServer, build_app
    (tmp_path / "text_encoder").mkdir()
    (tmp_path / "text_encoder" / "config.json").write_text(json.dumps(dict(
        vocab_size=300, hidden_size=24, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2,
        max_position_embeddings=16, layer_norm_eps=1e-5, hidden_act="quick_gelu", eos_token_id=2)))
    t5 = dict(T5, d_model=32)
    vae = dict(latent_channels=4, block_out_channels=[8, 16, 16, 16], layers_per_block=1, norm_num_groups=4,
               scaling_factor=0.36, shift_factor=0.11)
    srv = MultimodalServer("black-forest-labs/FLUX.1-dev", str(tmp_path), config_overrides={0: t5, 1: FLUX, 2: vae})
    try:
        assert srv.gs.stages[0].scheduler.pooled_model is not None
        with TestClient(build_app(srv)) as c:
            body = {"prompt": "a lighthouse at dusk", "size": "32x32", "num_inference_steps": 2, "seed": 3}
            r = c.post("/api/v1/images/generation", json=body)
            assert r.status_code == 200, r.text
            d = r.json()["data"]
            assert d["num_frames"] == 1 and d["width"] == 32
            assert c.post("/api/v1/images/generation", json=body).json()["data"]["b64_png"] == d["b64_png"]
            other = c.post("/api/v1/images/generation", json=dict(body, prompt="a harbour at dawn")).json()["data"]
            assert other["b64_png"] != d["b64_png"]
    finally:
        srv.shutdown()


def test_autoencoder_kl_names_shapes_and_roundtrip_scaling():
    from types import SimpleNamespace
    from sglang_jax_b200.multimodal.model_executor.loading import init_dummy
    from sglang_jax_b200.multimodal.models.vae import AutoencoderKL
    cfg = SimpleNamespace(latent_channels=4, block_out_channels=[8, 16, 32], layers_per_block=2, norm_num_groups=4,
                          scaling_factor=0.5, shift_factor=0.25, use_quant_conv=True, use_post_quant_conv=True)
    m = init_dummy(AutoencoderKL(cfg), seed=5, std=0.1).eval()
    names = {n for n, _ in m.named_parameters()}
    for n in ("encoder.conv_in.weight", "encoder.down_blocks.0.downsamplers.0.conv.weight",
              "encoder.down_blocks.1.resnets.0.conv_shortcut.weight", "encoder.mid_block.attentions.0.to_q.weight",
              "encoder.mid_block.attentions.0.group_norm.weight", "encoder.conv_out.bias", "quant_conv.weight",
              "post_quant_conv.bias", "decoder.up_blocks.0.resnets.2.conv2.weight",
              "decoder.up_blocks.1.upsamplers.0.conv.weight", "decoder.up_blocks.2.resnets.0.conv_shortcut.weight",
              "decoder.mid_block.resnets.1.norm2.weight", "decoder.conv_norm_out.weight"):
        assert n in names, n
    assert "encoder.down_blocks.2.downsamplers.0.conv.weight" not in names       # the last level keeps its size
    px = torch.rand(2, 3, 32, 24) * 2 - 1
    z = m.encode(px)
    assert z.shape == (2, 4, 8, 6) and m.spatial_factor == 4
    out = m.decode(z)
    assert out.shape == (2, 3, 32, 24) and out.abs().max() <= 1
    # scaling: decode undoes (x - shift) * scale before the decoder sees the latent
    raw = (z / 0.5 + 0.25)
    assert torch.allclose(m.decoder(m.post_quant_conv(raw)).clamp(-1, 1), out, atol=1e-6)
    vid = m.decode(torch.stack([z, z], dim=2))                                  # frames decode independently
    assert vid.shape == (2, 3, 2, 32, 24) and torch.allclose(vid[:, :, 0], out, atol=1e-6)
    sd = {k.replace(".to_q.", ".query."): v for k, v in m.state_dict().items()}
    m2 = AutoencoderKL(cfg)
    assert m2.load_weights(sd.items()) == names
    assert torch.allclose(m2.decode(z), out, atol=1e-6)


def test_qwen2_5_vl_image_prompt_matches_hf_through_the_engine(tmp_path):
    """ViT embeddings spliced over the image placeholders + 3-D rotary positions, served by the
    main scheduler (chunked prefill, a text-only request in the same batch) == HF generate."""
    from safetensors.torch import save_file
    from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration as HF
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.multimodal.manager.mrope_utils import get_rope_index
    from sglang_jax_b200.multimodal.models.qwen2_5_vl_vit import Qwen2_5_VisionTransformer
    from sglang_jax_b200.parallel import state as ps
    IMG, VS, VE = 290, 291, 292
    text = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=2, vocab_size=300, max_position_embeddings=512, rms_norm_eps=1e-6,
                tie_word_embeddings=False, rope_parameters={"rope_type": "default", "mrope_section": [2, 3, 3],
                                                            "rope_theta": 10000.0})
    vis = dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4,
               spatial_merge_size=2, temporal_patch_size=2, window_size=16, fullatt_block_indexes=[1],
               out_hidden_size=64, tokens_per_second=1)
    cfg = Qwen2_5_VLConfig(text_config=text, vision_config=vis, image_token_id=IMG, video_token_id=293,
                           vision_start_token_id=VS, vision_end_token_id=VE, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = HF(cfg).float().eval()
    for n, p in hf.named_parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.08)
        elif n.endswith("bias"):
            p.data.normal_(0, 0.02)
        else:
            p.data.uniform_(0.8, 1.2)
    hf.lm_head.weight.data.normal_(0, 0.5)                 # spread the logits so that greedy tokens vary
    path = tmp_path / "qwen25vl"
    path.mkdir()
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, str(path / "model.safetensors"))
    d = cfg.to_dict()
    d["architectures"] = ["Qwen2_5_VLForConditionalGeneration"]
    d["torch_dtype"] = "float32"
    (path / "config.json").write_text(json.dumps(d))
    grid = torch.tensor([[1, 4, 6]])                       # 24 patches -> 6 merged tokens
    px = torch.randn(24, 3 * 2 * 4 * 4, generator=torch.Generator().manual_seed(1))
    ids = [5, 9, 33, VS] + [IMG] * 6 + [VE, 41, 42, 7, 8]
    n_new = 8
    with torch.no_grad():
        # `mm_token_type_ids` is what makes the HF model compute the 3-D rotary positions itself
        want = hf.generate(input_ids=torch.tensor([ids]), pixel_values=px, image_grid_thw=grid,
                           mm_token_type_ids=(torch.tensor([ids]) == IMG).int(),
                           max_new_tokens=n_new, do_sample=False)[0, len(ids):].tolist()
        flat = hf.generate(input_ids=torch.tensor([ids]), pixel_values=px, image_grid_thw=grid,
                           max_new_tokens=n_new, do_sample=False)[0, len(ids):].tolist()
        assert flat != want                                   # the positions matter for this model
        want_text = hf.generate(input_ids=torch.tensor([[3, 4, 5, 6, 7, 8, 9]]), max_new_tokens=n_new,
                                do_sample=False)[0, 7:].tolist()
    vit = Qwen2_5_VisionTransformer(cfg.vision_config, dtype=torch.float32)
    vit.load_weights(hf.state_dict().items())
    img = vit(px, grid)
    assert img.shape == (6, 64)
    table = hf.state_dict()["model.language_model.embed_tokens.weight"]
    emb = table[torch.tensor(ids)].clone()
    emb[torch.tensor(ids) == IMG] = img
    pos, delta = get_rope_index(ids, image_grid_thw=grid, image_token_id=IMG, spatial_merge_size=2)
    assert pos[:, 3].tolist() == [3, 3, 3] and pos[:, 4].tolist() == [4, 4, 4] and pos[:, 9].tolist() == [4, 5, 6]
    assert pos[:, 10].tolist() == [7, 7, 7] and delta == 7 + 5 - len(ids)
    mm = {"input_embedding": emb, "mrope_positions": pos, "mrope_position_delta": delta}
    sp = {"max_new_tokens": n_new, "temperature": 0, "ignore_eos": True}
    for chunk in (None, 8):
        ps.reset_state()
        eng = Engine(model_path=str(path), device="cpu", dtype="float32", page_size=4, skip_tokenizer_init=True,
                     max_total_tokens=1024, enable_single_process=True, chunked_prefill_size=chunk)
        try:
            outs = eng.generate(input_ids=[ids, [3, 4, 5, 6, 7, 8, 9]], sampling_params=sp, mm_inputs=[mm, None])
            assert outs[0]["output_ids"] == want, (chunk, outs[0]["output_ids"], want)
            assert outs[1]["output_ids"] == want_text
            # the prefix cache is keyed by the media: the same image hits, another image (same token ids) does not
            again = eng.generate(input_ids=ids, sampling_params=sp, mm_inputs=mm)
            assert again["output_ids"] == want and again["meta_info"]["cached_tokens"] >= 12
            emb2 = emb.clone()
            emb2[torch.tensor(ids) == IMG] = img.flip(0)
            other = eng.generate(input_ids=ids, sampling_params=sp, mm_inputs=dict(mm, input_embedding=emb2))
            assert other["meta_info"]["cached_tokens"] == 0 and other["output_ids"] != want
            assert len(set(want)) >= 2
        finally:
            eng.shutdown()


def test_qwen3_omni_audio_encoder_matches_hf():
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeAudioEncoderConfig
    from transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe import Qwen3OmniMoeAudioEncoder as HF
    from sglang_jax_b200.multimodal.models.qwen3_omni.audio_encoder import Qwen3OmniMoeAudioEncoder, feat_lengths
    cfg = Qwen3OmniMoeAudioEncoderConfig(num_mel_bins=16, d_model=32, encoder_layers=2, encoder_attention_heads=4,
                                         encoder_ffn_dim=64, downsample_hidden_size=8, output_dim=24,
                                         max_source_positions=64, n_window=50, n_window_infer=200, conv_chunksize=4)
    torch.manual_seed(0)
    hf = HF._from_config(cfg, attn_implementation="eager").float().eval()
    for p in hf.parameters():
        p.data.normal_(0, 0.1) if p.dim() > 1 else p.data.uniform_(-0.2, 0.2)
    mine = Qwen3OmniMoeAudioEncoder(cfg, dtype=torch.float32).eval()
    assert mine.load_weights(hf.state_dict().items()) == {n for n, _ in mine.named_parameters()}
    # the HF port only windows its attention on the flash-attention path; one clip inside one window
    # is where its eager path and the windowed model agree
    lens = torch.tensor([157])
    feats = torch.randn(16, 157, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(feats, feature_lens=lens).last_hidden_state
    got = mine(feats, lens)
    assert got.shape == want.shape == (int(feat_lengths(lens).sum()), 24)
    assert torch.allclose(got, want, atol=2e-5), (got - want).abs().max()
    # clips packed together do not see each other, and a long clip attends within its windows
    lens2 = torch.tensor([157, 330])
    feats2 = torch.cat([feats, torch.randn(16, 330, generator=torch.Generator().manual_seed(2))], dim=1)
    both = mine(feats2, lens2)
    assert both.shape[0] == int(feat_lengths(lens2).sum())
    assert torch.allclose(both[: got.shape[0]], got, atol=1e-5)
    long_alone = mine(feats2[:, 157:], lens2[1:])
    assert torch.allclose(both[got.shape[0]:], long_alone, atol=1e-5)
    first_window = mine(feats2[:, 157:357], torch.tensor([200]))           # 200 frames = one attention window
    assert torch.allclose(long_alone[:26], first_window, atol=1e-5)


def test_qwen3_omni_vision_encoder_matches_hf():
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeVisionEncoderConfig
    from transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe import Qwen3OmniMoeVisionEncoder as HF
    from sglang_jax_b200.multimodal.models.qwen3_omni.vision_encoder import Qwen3OmniMoeVisionEncoder
    cfg = Qwen3OmniMoeVisionEncoderConfig(depth=3, hidden_size=32, intermediate_size=48, num_heads=4, in_channels=3,
                                          patch_size=4, spatial_merge_size=2, temporal_patch_size=2,
                                          out_hidden_size=40, num_position_embeddings=36,
                                          deepstack_visual_indexes=[0, 2], hidden_act="gelu_pytorch_tanh")
    torch.manual_seed(0)
    hf = HF._from_config(cfg, attn_implementation="sdpa").float().eval()
    for p in hf.parameters():
        p.data.normal_(0, 0.08) if p.dim() > 1 else p.data.uniform_(-0.3, 0.3)
    mine = Qwen3OmniMoeVisionEncoder(cfg, dtype=torch.float32).eval()
    assert mine.load_weights(hf.state_dict().items()) == {n for n, _ in mine.named_parameters()}
    grid = torch.tensor([[1, 6, 10], [2, 4, 4]])               # an image and a two-frame clip
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    px = torch.randn(n, 3 * 2 * 4 * 4, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(px, grid_thw=grid)
    got, deep = mine(px, grid, return_deepstack=True)
    assert got.shape == want.pooler_output.shape == (n // 4, 40)
    assert torch.allclose(got, want.pooler_output, atol=2e-4), (got - want.pooler_output).abs().max()
    assert len(deep) == 2
    for a, b in zip(deep, want.deepstack_features):
        assert torch.allclose(a, b, atol=2e-4)


def test_qwen3_omni_thinker_image_and_audio_prompt_matches_hf(tmp_path):
    """Audio + image + text prompt: my encoders feed the MoE language model (interleaved 3-stream
    rotary, deep-stack features after the first layers) through the engine == HF thinker generate."""
    from safetensors.torch import save_file
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeThinkerConfig
    from transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe import (
        Qwen3OmniMoeThinkerForConditionalGeneration as HF)
    from sglang_jax_b200 import Engine
    from sglang_jax_b200.multimodal.models.qwen3_omni.audio_encoder import Qwen3OmniMoeAudioEncoder, feat_lengths
    from sglang_jax_b200.multimodal.models.qwen3_omni.vision_encoder import Qwen3OmniMoeVisionEncoder
    from sglang_jax_b200.parallel import state as ps
    IMG, AUD = 290, 291
    text = dict(hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
                num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=300, num_experts=4,
                num_experts_per_tok=2, norm_topk_prob=True, max_position_embeddings=512, rms_norm_eps=1e-6,
                rope_parameters={"rope_type": "default", "mrope_section": [3, 3, 2], "rope_theta": 10000.0,
                                 "mrope_interleaved": True})
    vis = dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=4, in_channels=3, patch_size=4,
               spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=64, num_position_embeddings=36,
               deepstack_visual_indexes=[0, 1])
    aud = dict(num_mel_bins=16, d_model=32, encoder_layers=1, encoder_attention_heads=4, encoder_ffn_dim=64,
               downsample_hidden_size=8, output_dim=64, max_source_positions=64, n_window=50, n_window_infer=200)
    cfg = Qwen3OmniMoeThinkerConfig(text_config=text, vision_config=vis, audio_config=aud, image_token_id=IMG,
                                    audio_token_id=AUD, video_token_id=292, audio_start_token_id=293,
                                    vision_start_token_id=294, position_id_per_seconds=25)
    torch.manual_seed(0)
    hf = HF._from_config(cfg, attn_implementation="eager").float().eval()
    for n, p in hf.named_parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.08)
        elif n.endswith("bias"):
            p.data.normal_(0, 0.02)
        else:
            p.data.uniform_(0.8, 1.2)
    hf.lm_head.weight.data.normal_(0, 0.5)                 # spread the logits so that greedy tokens vary
    path = tmp_path / "omni"
    path.mkdir()
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, str(path / "model.safetensors"))
    d = cfg.to_dict()
    d.update(architectures=["Qwen3OmniMoeThinkerForConditionalGeneration"], torch_dtype="float32")
    (path / "config.json").write_text(json.dumps(d))
    grid = torch.tensor([[1, 4, 6]])
    px = torch.randn(24, 3 * 2 * 4 * 4, generator=torch.Generator().manual_seed(1))
    n_frames = 157
    n_aud = int(feat_lengths(torch.tensor([n_frames])))
    feats = torch.randn(1, 16, n_frames, generator=torch.Generator().manual_seed(2))
    ids = [5, 9, 293] + [AUD] * n_aud + [33, 294] + [IMG] * 6 + [41, 42, 7]
    n_new = 6
    inp = torch.tensor([ids])
    kw = dict(input_ids=inp, attention_mask=torch.ones_like(inp), pixel_values=px, image_grid_thw=grid,
              input_features=feats, feature_attention_mask=torch.ones(1, n_frames, dtype=torch.long))
    with torch.no_grad():
        want = hf.generate(**kw, max_new_tokens=n_new, do_sample=False)[0, len(ids):].tolist()
        pos, delta = hf.get_rope_index(inp, grid, None, torch.ones_like(inp), False, torch.tensor([n_frames]), None)
    assert len(set(want)) >= 2
    sd = hf.state_dict()
    vit = Qwen3OmniMoeVisionEncoder(cfg.vision_config, dtype=torch.float32)
    vit.load_weights(sd.items())
    enc = Qwen3OmniMoeAudioEncoder(cfg.audio_config, dtype=torch.float32)
    enc.load_weights(sd.items())
    img, deep = vit(px, grid, return_deepstack=True)
    audio = enc(feats[0], torch.tensor([n_frames]))
    t = torch.tensor(ids)
    emb = sd["model.embed_tokens.weight"][t].clone()
    emb[t == IMG], emb[t == AUD] = img, audio
    ds = torch.zeros(len(deep), len(ids), 64)
    for i, f in enumerate(deep):
        ds[i, t == IMG] = f
    mm = {"input_embedding": emb, "mrope_positions": pos[:, 0].numpy(), "mrope_position_delta": int(delta[0]),
          "deepstack": ds}
    from sglang_jax_b200.multimodal.manager.mrope_utils import get_rope_index
    my_pos, my_delta = get_rope_index(ids, image_grid_thw=grid, image_token_id=IMG, video_token_id=292,
                                      spatial_merge_size=2, tokens_per_second=25)
    assert (my_pos == pos[:, 0].long().numpy()).all() and my_delta == int(delta[0])
    sp = {"max_new_tokens": n_new, "temperature": 0, "ignore_eos": True}
    for chunk in (None, 16):
        ps.reset_state()
        eng = Engine(model_path=str(path), device="cpu", dtype="float32", page_size=4, skip_tokenizer_init=True,
                     max_total_tokens=1024, enable_single_process=True, chunked_prefill_size=chunk,
                     disable_radix_cache=True)
        try:
            out = eng.generate(input_ids=ids, sampling_params=sp, mm_inputs=mm)
            assert out["output_ids"] == want, (chunk, out["output_ids"], want)
        finally:
            eng.shutdown()
    # the same request through the two-stage pipeline (embedding stage -> serving engine) over HTTP
    from fastapi.testclient import TestClient
    from sglang_jax_b200.multimodal.entrypoint.http_server import MultimodalServer, build_app
    ps.reset_state()
    srv = MultimodalServer("Qwen/Qwen3-Omni-30B-A3B-Instruct", str(path),
                           config_overrides={1: dict(page_size=4, max_total_tokens=1024, tp_size=1),
                                             "media": dict(min_pixels=64, max_pixels=4096)})
    try:
        with TestClient(build_app(srv)) as c:
            assert [s["scheduler"] for s in c.get("/health").json()["stages"]] == ["embedding", "auto_regressive"]
            r = c.post("/v1/chat/completions", json={
                "input_ids": ids, "pixel_values": px.tolist(), "image_grid_thw": grid.tolist(),
                "audio_features": feats[0].tolist(), "max_tokens": n_new})
            assert r.status_code == 200, r.text
            assert r.json()["choices"][0]["message"]["output_ids"] == want
            # raw media: a PNG and PCM samples are preprocessed by the server, placeholders expanded
            from PIL import Image
            img = np.random.RandomState(0).randint(0, 255, (16, 24, 3), dtype=np.uint8)
            buf = io.BytesIO()
            Image.fromarray(img).save(buf, format="PNG")
            pcm = (np.sin(np.linspace(0, 300, 16000)) * 0.2).astype("<f4")
            short = [5, 9, 293, AUD, 33, 294, IMG, 41, 42, 7]
            r2 = c.post("/v1/chat/completions", json={
                "input_ids": short, "images": ["data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()],
                "audios": [base64.b64encode(pcm.tobytes()).decode()], "max_tokens": 4})
            assert r2.status_code == 200, r2.text
            assert len(r2.json()["choices"][0]["message"]["output_ids"]) == 4
            bad = c.post("/v1/chat/completions", json={"input_ids": [5, 9], "images": ["data:image/png;base64," +
                                                       base64.b64encode(buf.getvalue()).decode()]})
            assert bad.status_code == 400
    finally:
        srv.shutdown()


def test_kimi_k25_vision_tower_properties():
    from types import SimpleNamespace
    from sglang_jax_b200.multimodal.model_executor.loading import init_dummy
    from sglang_jax_b200.multimodal.models.kimi_k25.kimi_k25_vit import (KimiK25VisionModel, apply_rope_interleaved,
                                                                           rope_2d)
    cfg = SimpleNamespace(patch_size=4, in_channels=3, vt_hidden_size=32, vt_num_attention_heads=4,
                          vt_intermediate_size=48, vt_num_hidden_layers=2, init_pos_emb_height=6, init_pos_emb_width=6,
                          init_pos_emb_time=4, merge_kernel_size=[2, 2], text_hidden_size=40)
    m = init_dummy(KimiK25VisionModel(cfg, dtype=torch.float32), seed=2, std=0.1).eval()
    names = {n for n, _ in m.named_parameters()}
    for n in ("vision_tower.patch_embed.pos_emb.weight", "vision_tower.patch_embed.proj.bias",
              "vision_tower.encoder.blocks.1.wqkv.weight", "vision_tower.encoder.blocks.0.wo.bias",
              "vision_tower.encoder.blocks.0.mlp.fc0.weight", "vision_tower.encoder.blocks.0.norm1.weight",
              "vision_tower.encoder.final_layernorm.bias", "mm_projector.pre_norm.weight",
              "mm_projector.proj.0.weight", "mm_projector.proj.2.bias"):
        assert n in names, n
    g = torch.Generator().manual_seed(0)
    a = torch.randn(1 * 6 * 6, 3, 4, 4, generator=g)           # an image on the native grid
    b = torch.randn(2 * 4 * 8, 3, 4, 4, generator=g)           # a two-frame clip on a resized grid
    ya, yb = m(a, [[1, 6, 6]]), m(b, [[2, 4, 8]])
    assert ya.shape == (9, 40) and yb.shape == (8, 40)         # frames pooled, 2x2 patches merged
    both = m(torch.cat([a, b]), [[1, 6, 6], [2, 4, 8]])
    assert torch.allclose(both, torch.cat([ya, yb]), atol=1e-5)             # items never see each other
    assert torch.equal(m._abs_pos(1, 6, 6), m.vision_tower.patch_embed.pos_emb.weight.reshape(36, -1))
    assert m._abs_pos(2, 4, 8).shape == (64, 32)
    with pytest.raises(ValueError):
        m(torch.randn(5 * 4, 3, 4, 4), [[5, 2, 2]])
    # rotary: the origin is the identity, and q.k depends only on the (row, column) offset
    cos, sin = rope_2d(5, 7, 8)
    x = torch.randn(35, 1, 8, generator=g)
    assert torch.allclose(apply_rope_interleaved(x, cos, sin)[0], x[0])
    q, k = torch.randn(1, 1, 8, generator=g).expand(35, 1, 8), torch.randn(1, 1, 8, generator=g).expand(35, 1, 8)
    rq, rk = apply_rope_interleaved(q, cos, sin)[:, 0], apply_rope_interleaved(k, cos, sin)[:, 0]
    at = lambda r, c: r * 7 + c
    assert torch.allclose((rq[at(1, 2)] * rk[at(3, 5)]).sum(), (rq[at(2, 1)] * rk[at(4, 4)]).sum(), atol=1e-5)
    assert not torch.allclose((rq[at(1, 2)] * rk[at(3, 5)]).sum(), (rq[at(1, 2)] * rk[at(3, 6)]).sum(), atol=1e-4)
    sd = dict(m.state_dict())
    m2 = KimiK25VisionModel(cfg, dtype=torch.float32)
    assert m2.load_weights(sd.items()) == names
    assert torch.allclose(m2(a, [[1, 6, 6]]), ya)


MIMO_LOCAL = dict(group_size=2, audio_channels=2, local_dim=24, local_layers=1, local_attn_heads=2, local_head_dim=8,
                  local_ffn_dim=32, input_local_layers=1, input_local_dim=24, input_full_attention=True,
                  speech_vocab_sizes=[65, 65], speech_empty_ids=[64, 64], delay_pattern=[0, 1], attention_bias=True,
                  rope_theta=10000.0, rms_norm_eps=1e-6)


def test_mimo_audio_local_transformers():
    from types import SimpleNamespace
    from sglang_jax_b200.multimodal.model_executor.loading import init_dummy
    from sglang_jax_b200.multimodal.models.mimo_audio_backbone import MiMoAudioLocalModules
    m = init_dummy(MiMoAudioLocalModules(SimpleNamespace(hidden_size=32, **MIMO_LOCAL), dtype=torch.float32), 3, 0.2).eval()
    names = {n for n, _ in m.named_parameters()}
    for n in ("local_transformer.layers.0.self_attn.q_proj.bias", "input_local_transformer.layers.0.mlp.down_proj.weight",
              "local_transformer.norm.weight", "speech_embeddings.1.weight", "local_transformer_lm_heads.0.weight",
              "speech_group_downcast.weight", "hidden_states_downcast.weight"):
        assert n in names, n
    ids = torch.tensor([[[3, 4], [5, 6]], [[7, 8], [9, 10]], [[64, 64], [64, 64]]])
    e = m.group_embeds(ids, torch.tensor([True, True, False]))
    assert e.shape == (3, 32) and bool((e[2] == 0).all()) and not torch.allclose(e[0], e[1])
    # the patch encoder is bidirectional: the second frame changes the first frame's contribution
    swapped = m.group_embeds(ids[:1].flip(1), torch.tensor([True]))
    assert not torch.allclose(swapped, e[:1])
    # groups are independent of one another
    assert torch.allclose(m.group_embeds(ids[1:2], torch.tensor([True])), e[1:2], atol=1e-6)
    h = torch.randn(2, 32, generator=torch.Generator().manual_seed(0))
    codes = m.patch_decode(h)
    assert codes.shape == (2, 2, 2) and int(codes.max()) < 64                    # never the `empty` code
    assert torch.equal(codes, m.patch_decode(h)) and torch.equal(m.patch_decode(h[:1]), codes[:1])
    # the decoder's cache matters: with the delay pattern, channel 1 of frame 0 is produced at local step 1
    # and must depend on channel 0 of frame 0 (fed back at step 1) — change that embedding and it moves
    before = m.patch_decode(h[:1])
    m.speech_embeddings[0].weight.data[int(before[0, 0, 0])] += 5.0
    after = m.patch_decode(h[:1])
    assert int(after[0, 0, 0]) == int(before[0, 0, 0])
    assert not torch.equal(after[0, :, 1], before[0, :, 1]) or not torch.equal(after[0, 1], before[0, 1])


def test_mimo_audio_grouped_backbone_pipeline(tmp_path):
    """audio -> codec tokens -> grouped MiMo backbone (patch encoder in, patch decoder out) -> codec -> wave."""
    from fastapi.testclient import TestClient
    from sglang_jax_b200.multimodal.entrypoint.http_server import MultimodalServer, build_app
    llm_cfg = dict(architectures=["MiMoAudioForCausalLM"], model_type="qwen2", hidden_size=32, intermediate_size=64,
                   num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=320,
                   max_position_embeddings=256, tie_word_embeddings=False, torch_dtype="float32", **MIMO_LOCAL)
    path = tmp_path / "mimo_audio"
    path.mkdir()
    (path / "config.json").write_text(json.dumps(llm_cfg))
    codec = dict(sample_rate=8000, n_mels=20, d_model=32, heads=2, layers=1, num_quantizers=2, codebook_size=64, hop=80)
    srv = MultimodalServer("XiaomiMiMo/MiMo-Audio", None, config_overrides={
        0: codec, 1: {"model_path": str(path), "load_format": "dummy", "empty_idx": 300}, 2: codec})
    try:
        bb = srv.gs.stages[1].scheduler
        assert bb.local is not None and bb.local.group == 2
        with TestClient(build_app(srv)) as c:
            wave = np.sin(np.linspace(0, 200, 4000)).astype("<f4")
            asr = c.post("/v1/audio/transcriptions", json={"audio_b64": base64.b64encode(wave.tobytes()).decode(),
                                                           "max_new_tokens": 5})
            assert asr.status_code == 200, asr.text
            tts = c.post("/v1/audio/speech", json={"input": "hello", "max_new_tokens": 6})
            assert tts.status_code == 200 and tts.content[:4] == b"RIFF"
            again = c.post("/v1/audio/speech", json={"input": "hello", "max_new_tokens": 6})
            assert again.content == tts.content
            longer = c.post("/v1/audio/speech", json={"input": "hello", "max_new_tokens": 9})
            assert len(longer.content) > len(tts.content)            # 2 frames of audio per generated group
    finally:
        srv.shutdown()


def test_media_preprocessing_matches_hf_processors():
    from PIL import Image
    from transformers import WhisperFeatureExtractor
    from transformers.models.qwen2_vl.image_processing_qwen2_vl import Qwen2VLImageProcessor
    from sglang_jax_b200.multimodal.manager.processors import (expand_placeholders, frames_to_patches, load_image,
                                                                 log_mel_spectrogram, smart_resize)
    rng = np.random.RandomState(0)
    img = rng.randint(0, 255, (75, 131, 3), dtype=np.uint8)
    hf = Qwen2VLImageProcessor(patch_size=14, merge_size=2, temporal_patch_size=2, min_pixels=56 * 56,
                               max_pixels=28 * 28 * 64)
    want = hf(images=[Image.fromarray(img)], return_tensors="np")
    px, grid = frames_to_patches(img[None], 14, 2, 2, min_pixels=56 * 56, max_pixels=28 * 28 * 64)
    assert list(grid) == want["image_grid_thw"][0].tolist()
    assert px.shape == want["pixel_values"].shape
    assert np.abs(px - want["pixel_values"]).max() < 0.03               # bicubic resampling rounds pixels differently
    exact = rng.randint(0, 255, (56, 84, 3), dtype=np.uint8)            # already on the patch grid: no resampling
    w2 = hf(images=[Image.fromarray(exact)], return_tensors="np")
    p2, g2 = frames_to_patches(exact[None], 14, 2, 2, min_pixels=56 * 56, max_pixels=28 * 28 * 64)
    assert list(g2) == [1, 4, 6] and np.allclose(p2, w2["pixel_values"], atol=1e-5)
    assert smart_resize(75, 131, 28, 56 * 56, 28 * 28 * 64) == (84, 140)
    buf = io.BytesIO()
    Image.fromarray(exact).save(buf, format="PNG")
    uri = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    assert np.array_equal(load_image(uri), exact)
    wave = (np.sin(np.linspace(0, 900, 16000 * 2)) * 0.3 + rng.randn(32000) * 0.01).astype(np.float32)
    fe = WhisperFeatureExtractor(feature_size=128, sampling_rate=16000, hop_length=160, n_fft=400)
    ref = fe(wave, sampling_rate=16000, return_tensors="np", padding="do_not_pad" if False else "longest")["input_features"][0]
    got = log_mel_spectrogram(wave, 16000, 400, 160, 128).numpy()
    n = got.shape[1]
    assert n == 200 and np.abs(got - ref[:, :n]).max() < 2e-3
    assert expand_placeholders([1, 9, 2, 9, 3], 9, [3, 1]) == [1, 9, 9, 9, 2, 9, 3]
    with pytest.raises(ValueError):
        expand_placeholders([1, 9], 9, [1, 2])


def test_wan_vae_encoder_decoder_with_feature_cache():
    """The full Wan video VAE: 1 + 4k frames <-> 1 + k latent frames (8x in space), processed in chunks with cached
    convolution tails.  Causality makes the chunked pass prefix-stable: the latents of a longer clip start with the
    latents of its prefix, and so do the decoded frames."""
    from types import SimpleNamespace
    import torch
    from sglang_jax_b200.multimodal.models.wan_vae import WanVAE
    torch.manual_seed(0)
    cfg = SimpleNamespace(base_dim=8, z_dim=4, dim_mult=(1, 2, 4, 4), num_res_blocks=1,
                          temporal_downsample=(False, True, True), latents_mean=[0.1, -0.2, 0.0, 0.3],
                          latents_std=[1.5, 0.5, 1.0, 2.0])
    vae = WanVAE(cfg).eval()
    for p in vae.parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.15)
    video = torch.rand(1, 3, 9, 32, 32) * 2 - 1
    z9 = vae.encode(video)
    assert z9.shape == (1, 4, 3, 4, 4)
    z5 = vae.encode(video[:, :, :5])
    z1 = vae.encode(video[:, :, :1])
    assert z5.shape == (1, 4, 2, 4, 4) and z1.shape == (1, 4, 1, 4, 4)
    assert torch.allclose(z9[:, :, :2], z5, atol=1e-5) and torch.allclose(z9[:, :, :1], z1, atol=1e-5)
    other = video.clone()
    other[:, :, 5:] = 0.5                                    # later frames differ: earlier latents must not move
    assert torch.allclose(vae.encode(other)[:, :, :2], z9[:, :, :2], atol=1e-5)
    assert not torch.allclose(vae.encode(other)[:, :, 2], z9[:, :, 2], atol=1e-3)
    out = vae.decode(z9)
    assert out.shape == (1, 3, 9, 32, 32) and out.abs().max() <= 1.0
    out5 = vae.decode(z9[:, :, :2])
    assert out5.shape == (1, 3, 5, 32, 32) and torch.allclose(out[:, :, :5], out5, atol=1e-5)
    assert vae.decode(z9[:, :, :1]).shape == (1, 3, 1, 32, 32)
    # the latent normalisation is undone by decode: scaling statistics cancel
    raw = WanVAE(SimpleNamespace(**{**cfg.__dict__, "latents_mean": None, "latents_std": None})).eval()
    raw.load_state_dict(vae.state_dict())
    zr = raw.encode(video)
    mean, std = torch.tensor(cfg.latents_mean).view(1, 4, 1, 1, 1), torch.tensor(cfg.latents_std).view(1, 4, 1, 1, 1)
    assert torch.allclose((zr - mean) / std, z9, atol=1e-5) and torch.allclose(raw.decode(zr), out, atol=1e-5)
    # checkpoint tensors load by name
    names = set(n for n, _ in vae.named_parameters())
    assert {"encoder.conv_in.weight", "encoder.down_blocks.0.norm1.gamma", "encoder.mid_block.attentions.0.to_qkv.weight",
            "quant_conv.weight", "post_quant_conv.weight", "decoder.up_blocks.0.upsamplers.0.time_conv.weight",
            "decoder.up_blocks.2.upsamplers.0.resample.1.weight", "decoder.conv_out.bias"} <= names
    fresh = WanVAE(cfg).eval()
    assert fresh.load_weights(vae.state_dict().items()) == names
    assert torch.allclose(fresh.encode(video), z9, atol=1e-6)
