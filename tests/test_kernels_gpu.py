"""Numerics of every sm_100a kernel against the plain-PyTorch fp32 statement of the same op."""

import math

import pytest
import torch

from sglang_jax_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def native():
    from sglang_jax_b200.ops import native
    native.lib()
    yield native
    torch.cuda.synchronize()
    native.check_status()


def _bf16(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


def _close(a, b, atol, rtol):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = (err > tol).float().mean().item()
    assert bad < 1e-4, f"max err {err.max().item():.4g}, {bad * 100:.3f}% outside tol"


@pytest.mark.parametrize("T,H", [(1, 256), (7, 5120), (128, 5120), (33, 8192), (5, 2048)])
def test_rmsnorm(native, T, H):
    x, w = _bf16(T, H, seed=1), _bf16(H, seed=2) * 0.1 + 1
    _close(native.rmsnorm(x, w, 1e-6), ref.rmsnorm(x.float(), w.float(), 1e-6), 2e-2, 2e-2)
    r = _bf16(T, H, seed=3)
    r2 = r.clone()
    y, rout = native.fused_add_rmsnorm(x, r2, w, 1e-6)
    ey, er = ref.fused_add_rmsnorm(x, r, w, 1e-6)
    assert torch.equal(rout, er)
    _close(y, ey, 2e-2, 2e-2)


@pytest.mark.parametrize("T,I", [(1, 512), (130, 25600), (4096, 3200)])
def test_silu_and_mul(native, T, I):
    x = _bf16(T, 2 * I, seed=4)
    _close(native.silu_and_mul(x), ref.silu_and_mul(x.float()), 1e-2, 2e-2)


def test_embedding_argmax(native):
    table = _bf16(1000, 256, seed=5)
    ids = torch.randint(0, 1000, (77,), device="cuda", dtype=torch.int32)
    assert torch.equal(native.embedding(ids, table), table[ids.long()])
    assert torch.equal(native.embedding(ids, table[100:600].contiguous(), 100, True),
                       ref.embedding(ids, table[100:600], 100, True))
    for dt in (torch.float32, torch.bfloat16):
        logits = torch.randn(9, 151936, device="cuda").to(dt)
        logits[3, 77] = logits[3, 5000] = 100.0     # tie: first index wins
        assert torch.equal(native.argmax(logits).long(), torch.argmax(logits.float(), dim=-1))


@pytest.mark.parametrize("M,N,K", [
    (1, 512, 256), (8, 5120, 5120), (16, 1024, 4096), (33, 6400, 5120), (128, 5120, 8192),
    (128, 10240, 5120), (200, 2048, 1024), (256, 512, 25600),
    (257, 512, 512), (512, 5120, 5120), (1000, 768, 2048), (4096, 5120, 3200), (300, 1032, 264),
])
def test_gemm(native, M, N, K):
    x = _bf16(M, K, seed=6)
    w = _bf16(N, K, scale=0.05, seed=7)
    b = _bf16(N, seed=8)
    expect = x.float() @ w.float().t()
    got = native.linear(x, w)
    torch.cuda.synchronize()
    native.check_status()
    tol = 0.02 * math.sqrt(K) * 0.05 + 0.02
    _close(got, expect, tol, 1.5e-2)
    _close(native.linear(x, w, b), expect + b.float(), tol, 1.5e-2)


@pytest.mark.parametrize("mode,splits", [(0, 1), (1, 1), (1, 2), (1, 5)])
def test_gemm_forced_modes(native, mode, splits):
    M, N, K = 96, 1024, 4096
    x, w = _bf16(M, K, seed=9), _bf16(N, K, scale=0.05, seed=10)
    got = native.linear(x, w, None, force_mode=mode, force_splits=splits)
    torch.cuda.synchronize()
    native.check_status()
    _close(got, x.float() @ w.float().t(), 0.1, 1.5e-2)
    # split-K leaves its tile counters clean
    assert int(native.gemm_scratch(x.device).counters.abs().sum().item()) == 0


def _make_cache(num_pages, Hkv, P, D, seed):
    return _bf16(num_pages, 2, Hkv, P, D, seed=seed)


@pytest.mark.parametrize("D,Hq,Hkv,qk_norm,neox", [(128, 8, 2, True, True), (128, 4, 4, False, True),
                                                   (64, 4, 2, True, True), (128, 8, 1, False, False)])
def test_rope_kvwrite(native, D, Hq, Hkv, qk_norm, neox):
    T, P, pages = 37, 16, 12
    qkv = _bf16(T, (Hq + 2 * Hkv) * D, seed=11)
    pos = torch.randint(0, 4000, (T,), device="cuda", dtype=torch.int32)
    loc = (torch.randperm((pages - 1) * P, device="cuda")[:T] + P).to(torch.int32)
    cs = ref.build_cos_sin_cache(D, 4096, 1e6, device="cuda")
    qw = (_bf16(D, seed=12) * 0.1 + 1) if qk_norm else None
    kw = (_bf16(D, seed=13) * 0.1 + 1) if qk_norm else None
    c1, c2 = torch.zeros(pages, 2, Hkv, P, D, device="cuda", dtype=torch.bfloat16), None
    c2 = c1.clone()
    q1 = native.rope_qknorm_kvwrite(qkv, pos, cs, qw, kw, 1e-6, Hq, Hkv, D, c1, loc, P, neox)
    q2 = ref.rope_qknorm_kvwrite(qkv, pos, cs, qw, kw, 1e-6, Hq, Hkv, D, c2, loc, P, neox)
    _close(q1, q2, 3e-2, 2e-2)
    _close(c1, c2, 3e-2, 2e-2)


def _attn_setup(B, seqs, P, Hkv, D, seed=0):
    pages_per = [(s + P - 1) // P for s in seqs]
    num_pages = sum(pages_per) + 3
    cache = _make_cache(num_pages, Hkv, P, D, seed)
    max_pages = max(pages_per) + 2
    pt = torch.zeros(B + 3, max_pages, dtype=torch.int32, device="cuda")
    perm = (torch.randperm(num_pages - 1, device="cuda") + 1).to(torch.int32)
    o = 0
    rows = torch.randperm(B + 2, device="cuda")[:B].to(torch.int32)
    for b in range(B):
        pt[rows[b], :pages_per[b]] = perm[o:o + pages_per[b]]
        o += pages_per[b]
    return cache, pt, rows


@pytest.mark.parametrize("P", [16, 64, 128])
@pytest.mark.parametrize("Hq,Hkv,D", [(8, 1, 128), (16, 4, 128), (4, 2, 64)])
def test_paged_decode(native, P, Hq, Hkv, D):
    seqs = [1, 17, 64, 65, 300, 1000, 129, 2047]
    B = len(seqs)
    cache, pt, rows = _attn_setup(B, seqs, P, Hkv, D, seed=20)
    q = _bf16(B, Hq, D, seed=21)
    sl = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    scale = D ** -0.5
    expect = ref.paged_attention(q.float(), cache.float(), pt, rows, sl, P, scale)
    for splits in (1, 3, None):
        got = native.paged_attention(q, cache, pt, rows, sl, P, scale, max_seq_len=max(seqs), num_splits=splits)
        torch.cuda.synchronize()
        native.check_status()
        _close(got, expect, 2e-2, 2e-2)
    got = native.paged_attention(q, cache, pt, rows, sl, P, scale, sliding_window=100, max_seq_len=max(seqs))
    _close(got, ref.paged_attention(q.float(), cache.float(), pt, rows, sl, P, scale, sliding_window=100), 2e-2, 2e-2)
    got = native.paged_attention(q, cache, pt, rows, sl, P, scale, soft_cap=30.0, max_seq_len=max(seqs))
    _close(got, ref.paged_attention(q.float(), cache.float(), pt, rows, sl, P, scale, soft_cap=30.0), 2e-2, 2e-2)


@pytest.mark.parametrize("P", [16, 64])
@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 4, 64)])
def test_paged_extend(native, P, Hq, Hkv, D):
    prefix = [0, 64, 5, 130, 0, 1]
    ext = [1, 63, 64, 200, 513, 17]
    seqs = [a + b for a, b in zip(prefix, ext)]
    B = len(seqs)
    cache, pt, rows = _attn_setup(B, seqs, P, Hkv, D, seed=30)
    T = sum(ext)
    q = _bf16(T, Hq, D, seed=31)
    sl = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    pl = torch.tensor(prefix, dtype=torch.int32, device="cuda")
    cu = torch.zeros(B + 1, dtype=torch.int32, device="cuda")
    cu[1:] = torch.tensor(ext, device="cuda").cumsum(0)
    scale = D ** -0.5
    got = native.paged_attention(q, cache, pt, rows, sl, P, scale, cu, pl)
    torch.cuda.synchronize()
    native.check_status()
    _close(got, ref.paged_attention(q.float(), cache.float(), pt, rows, sl, P, scale, cu, pl), 2e-2, 2e-2)
    got = native.paged_attention(q, cache, pt, rows, sl, P, scale, cu, pl, sliding_window=70)
    _close(got, ref.paged_attention(q.float(), cache.float(), pt, rows, sl, P, scale, cu, pl, sliding_window=70),
           2e-2, 2e-2)


@pytest.mark.parametrize("E,k,scoring,groups,topk_group,bias,renorm", [
    (128, 8, "softmax", 0, 0, False, True), (64, 4, "softmax", 0, 0, False, False),
    (256, 8, "sigmoid", 8, 4, True, True), (256, 8, "sigmoid", 8, 4, False, True), (16, 2, "tanh", 0, 0, False, True),
])
def test_topk_route(native, E, k, scoring, groups, topk_group, bias, renorm):
    from sglang_jax_b200.ops import moe_native
    g = torch.Generator(device="cuda").manual_seed(40)
    logits = torch.randn(77, E, device="cuda", generator=g)
    b = torch.randn(E, device="cuda", generator=g) * 0.1 if bias else None
    w, ids = moe_native.topk_route(logits, k, scoring, renorm, b, groups, topk_group, 2.5)
    ew, eids = ref.topk_route(logits, k, scoring, renorm, b, groups, topk_group, 2.5)
    assert torch.equal(ids.sort(-1).values, eids.sort(-1).values)
    order, eorder = ids.argsort(-1), eids.argsort(-1)
    torch.testing.assert_close(w.gather(1, order), ew.gather(1, eorder), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("T,E,E_local,e0,k,H,I", [
    (5, 16, 16, 0, 2, 256, 128), (40, 32, 8, 8, 4, 512, 384), (128, 128, 16, 32, 8, 2048, 768),
    (700, 32, 32, 0, 4, 512, 256), (1500, 64, 16, 16, 8, 1024, 768),
])
def test_fused_experts(native, T, E, E_local, e0, k, H, I):
    from sglang_jax_b200.ops import moe_native
    x = _bf16(T, H, seed=50)
    w13 = _bf16(E_local, 2 * I, H, scale=0.05, seed=51)
    w2 = _bf16(E_local, H, I, scale=0.05, seed=52)
    logits = torch.randn(T, E, device="cuda", generator=torch.Generator(device="cuda").manual_seed(53))
    tw, ids = ref.topk_route(logits, k)
    got = moe_native.fused_experts(x, w13, w2, tw, ids, e0)
    torch.cuda.synchronize()
    native.check_status()
    exp = ref.moe_forward(x.float(), w13.float(), w2.float(), tw, ids, e0)
    _close(got, exp, 3e-2, 3e-2)


@pytest.mark.parametrize("T,K,gated", [(7, 512, False), (130, 5120, False), (33, 768, True), (3, 25600, False), (64, 2048, True)])
def test_quant_fp8_rows(native, T, K, gated):
    """Per-token e4m3 quantisation kernel (plain and fused SiLU-gate) vs the PyTorch statement."""
    from sglang_jax_b200.utils.quantization import quantize_activation
    x = _bf16(T, 2 * K if gated else K, scale=3.0, seed=72)
    x[0, :8] = 0.0
    a = torch.nn.functional.silu(x[:, :K].float()) * x[:, K:].float() if gated else x.float()
    q, s = native.quant_fp8_rows(x, gated=gated)
    torch.cuda.synchronize()
    eq, es = quantize_activation(a, torch.float8_e4m3fn)
    torch.testing.assert_close(s, es.view(-1), rtol=2e-3 if gated else 1e-6, atol=0)
    back, want = q.float() * s[:, None], eq.float() * es
    assert q.dtype == torch.float8_e4m3fn and torch.isfinite(back).all()
    # one e4m3 step (2^-3 relative) at most where a rounding boundary fell the other way
    assert ((back - want).abs() <= 0.126 * want.abs() + 1e-6 + s[:, None] * 2 ** -9).all()
    assert ((back - want).abs() > 1e-6).float().mean().item() < (0.02 if gated else 1e-3)
    valid = torch.tensor([T // 2], dtype=torch.int32, device="cuda")
    q2, s2 = native.quant_fp8_rows(x, gated=gated, valid_rows=valid)
    assert torch.equal(q2[: T // 2].view(torch.uint8), q[: T // 2].view(torch.uint8))


@pytest.mark.parametrize("T,E,E_local,e0,k,H,I", [
    (5, 16, 16, 0, 2, 256, 128), (40, 32, 8, 8, 4, 512, 384), (128, 128, 16, 32, 8, 2048, 768),
    (700, 32, 32, 0, 4, 512, 256), (1500, 64, 16, 16, 8, 1024, 768),
])
def test_fused_experts_fp8(native, T, E, E_local, e0, k, H, I):
    """W8A8 e4m3 expert FFN (grouped fp8 tcgen05 GEMMs, decode and prefill tilings, expert-parallel slices)
    vs the PyTorch statement on the same quantised weights, and near the unquantised bf16 result."""
    from sglang_jax_b200.layers.moe import FusedMoE, _fp8_reference_experts
    moe = FusedMoE(E, H, I, tp_size=E // E_local, tp_rank=e0 // E_local, ep_size=E // E_local).cuda()
    assert moe.num_local_experts == E_local and moe.expert_start == e0
    moe.w13_weight.data.copy_(_bf16(E_local, 2 * I, H, scale=0.05, seed=51))
    moe.w2_weight.data.copy_(_bf16(E_local, H, I, scale=0.05, seed=52))
    x = _bf16(T, H, seed=50)
    logits = torch.randn(T, E, device="cuda", generator=torch.Generator(device="cuda").manual_seed(53))
    tw, ids = ref.topk_route(logits, k)
    full = ref.moe_forward(x.float(), moe.w13_weight.float(), moe.w2_weight.float(), tw, ids, e0)
    moe.quantize_(torch.float8_e4m3fn, None, torch.float8_e4m3fn)
    assert moe.fp8 and moe.w13_weight.dtype == torch.float8_e4m3fn and moe.w13_scale.shape == (E_local, 2 * I)
    got = moe(x, tw, ids)
    torch.cuda.synchronize()
    native.check_status()
    want = _fp8_reference_experts(x, moe, tw, ids)
    assert ((got.float() - want.float()).norm() / want.float().norm()).item() < 0.02
    _close(got, want, 6e-2, 6e-2)
    assert ((got.float() - full).norm() / full.norm()).item() < 0.1


def _filtered_probs_f64(logits, temps, ks, ps, mps):
    """Sort-based statement of temperature / top-k / top-p / min-p in float64 (fp32 cumulative sums over a
    150k vocabulary drift by more than the spacing of the top-p boundary)."""
    x = logits.double() / temps.double().view(-1, 1).clamp_min(1e-6)
    probs = torch.softmax(x, dim=-1)
    sp, si = probs.sort(dim=-1, descending=True)
    V = probs.shape[-1]
    keep = torch.arange(V, device=probs.device).view(1, -1) < ks.long().view(-1, 1).clamp(max=V)
    keep &= (sp.cumsum(-1) - sp) < ps.double().view(-1, 1)
    keep &= sp >= sp[:, :1] * mps.double().view(-1, 1)
    keep[:, 0] = True
    sp = sp * keep
    sp = sp / sp.sum(-1, keepdim=True)
    return torch.zeros_like(probs).scatter_(1, si, sp).float()


@pytest.mark.parametrize("B,V,dtype", [(24, 151936, torch.float32), (16, 5003, torch.float32), (12, 32000, torch.bfloat16)])
def test_sample_filtered_matches_sorted_reference(native, B, V, dtype):
    """Radix-select top-k / top-p / min-p + hashed Gumbel draw vs the sort-based PyTorch statement: same kept
    set and probabilities, same seeded draw, greedy rows return the argmax."""
    g = torch.Generator(device="cuda").manual_seed(80)
    logits = (torch.randn(B, V, device="cuda", generator=g) * 3).to(dtype)
    temps = torch.rand(B, device="cuda", generator=g) + 0.5
    ks = torch.randint(2, 300, (B,), device="cuda", generator=g, dtype=torch.int32)
    ks[::4] = V + 7                                         # top-k off
    ks[5] = 1                                               # greedy row
    ps = torch.rand(B, device="cuda", generator=g) * 0.8 + 0.2
    ps[1::4] = 1.0                                          # top-p off
    mps = torch.rand(B, device="cuda", generator=g) * 0.05
    mps[::2] = 0.0
    ks[2], ps[2], mps[2] = V, 1.0, 0.0                      # no filter at all
    ks[3], ps[3], mps[3] = V, 1.0, 0.02                     # min-p alone
    seeds = torch.randint(0, 2 ** 31 - 1, (B,), device="cuda", generator=g, dtype=torch.int32)
    pos = torch.randint(0, 4096, (B,), device="cuda", generator=g, dtype=torch.int32)
    ids, probs = native.sample_filtered(logits, temps, ks, ps, mps, seeds, pos, return_probs=True)
    torch.cuda.synchronize()
    want = _filtered_probs_f64(logits, temps, ks, ps, mps)
    live = ks > 1
    assert torch.equal(ids[~live].long(), logits[~live].float().argmax(-1))
    torch.testing.assert_close(probs[live].sum(-1), torch.ones(int(live.sum()), device="cuda"), rtol=1e-4, atol=1e-4)
    if dtype == torch.float32:
        # a top-p close to 1 puts the boundary among tokens of ~1e-9 probability, where the last bits of the
        # kernel's fast exp move it by many (negligible) tokens: compare by mass, and exactly on the small vocabulary
        flips = (probs[live] > 0) != (want[live] > 0)
        assert float(((probs[live] + want[live]) * flips).sum(-1).max()) < 2e-5
        assert float((probs[live] - want[live]).abs().sum(-1).max()) < 2e-4
        same = flips.sum(-1) == 0
        torch.testing.assert_close(probs[live][same], want[live][same], rtol=2e-3, atol=1e-7)
        if V < 10000:
            assert bool(same.all())
    else:                                                   # bf16 rows are full of ties: all of them are kept
        assert bool(((want[live] > 0) <= (probs[live] > 0)).all())
        tie_free = (probs[live] > 0).sum(-1) == (want[live] > 0).sum(-1)
        torch.testing.assert_close(probs[live][tie_free], want[live][tie_free], rtol=2e-3, atol=1e-7)
    assert bool((probs[live].gather(1, ids[live].long().view(-1, 1)) > 0).all())
    drawn = ref.multinomial_with_seed(probs, seeds, pos)
    assert (drawn[live] == ids[live].long()).float().mean().item() >= 0.9
    again = native.sample_filtered(logits, temps, ks, ps, mps, seeds, pos)
    assert torch.equal(again, ids)                          # bit-reproducible
    other = native.sample_filtered(logits, temps, ks, ps, mps, seeds + 1, pos)
    assert not torch.equal(other[live], ids[live])


def test_sample_filtered_follows_the_distribution(native):
    """Many rows of one small distribution with different seeds, unseeded-request hash: empirical frequencies
    match the filtered probabilities (top-p removes the tail)."""
    base = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, -3.0, -3.5, -8.0], device="cuda")
    B = 20000
    logits = base.repeat(B, 1)
    one = lambda v, dt=torch.float32: torch.full((B,), v, device="cuda", dtype=dt)
    seeds = torch.arange(B, device="cuda", dtype=torch.int32) * 7919 + 13
    pos = torch.arange(B, device="cuda", dtype=torch.int32) % 97
    ids = native.sample_filtered(logits, one(0.8), one(8, torch.int32), one(0.9), one(0.0), seeds, pos,
                                 request_seeded=False)
    want = ref.top_k_top_p_min_p_probs(base.view(1, -1), one(0.8)[:1], one(8, torch.int64)[:1], one(0.9)[:1], one(0.0)[:1])[0]
    freq = torch.bincount(ids.long(), minlength=8).float() / B
    assert bool((freq[want == 0] == 0).all()) and int((want > 0).sum()) < 8
    torch.testing.assert_close(freq, want, rtol=0.0, atol=0.015)


def test_sampler_module_uses_the_sampling_kernel(native):
    """`Sampler.forward` on the GPU: seeded requests reproduce the PyTorch statement of the same draw, unseeded
    ones are reproducible per sampler seed, vary between steps and stay inside the top-k set."""
    from types import SimpleNamespace
    from sglang_jax_b200 import ops
    from sglang_jax_b200.layers.sampler import Sampler, SamplingMetadata
    B, V = 32, 4096
    g = torch.Generator(device="cuda").manual_seed(90)
    logits = torch.randn(B, V, device="cuda", generator=g) * 2
    ks = torch.full((B,), 5, device="cuda", dtype=torch.int32)
    ks[7] = 1
    meta = SamplingMetadata(temperatures=torch.full((B,), 0.9, device="cuda"), top_ks=ks,
                            top_ps=torch.full((B,), 0.95, device="cuda"), min_ps=torch.zeros(B, device="cuda"),
                            is_all_greedy=False, need_filter=True,
                            sampling_seeds=torch.arange(B, device="cuda", dtype=torch.int32) + 100,
                            positions=torch.arange(B, device="cuda", dtype=torch.int32))
    out = SimpleNamespace(next_token_logits=logits)
    ids = Sampler()(out, meta)
    ops.set_force_reference(True)
    try:
        want = Sampler()(out, meta)
    finally:
        ops.set_force_reference(False)
    assert ids.dtype == torch.int32 and (ids == want).float().mean().item() >= 0.9   # fast log vs libm at near-ties
    assert int(ids[7]) == int(logits[7].argmax())
    meta.sampling_seeds = None
    a, b = Sampler(rng_seed=3), Sampler(rng_seed=3)
    first, second = a(out, meta), a(out, meta)
    assert torch.equal(first, b(out, meta)) and not torch.equal(first, second)
    top5 = logits.topk(5, dim=-1).indices
    assert bool((top5 == first.long().view(-1, 1)).any(-1).all())


@pytest.mark.parametrize("Hq,Hkv,D,lens", [(4, 4, 128, [5, 64, 130, 0, 700]), (16, 16, 80, [37, 256, 100]),
                                            (8, 2, 64, [1, 63, 65, 129]), (6, 6, 72, [300])])
def test_varlen_bidirectional_attention(native, Hq, Hkv, D, lens):
    """Packed encoder attention (no causal rule) through the paged extend kernel, head dims padded to 64 / 128,
    vs an fp32 softmax per sequence."""
    T = sum(lens)
    q, k, v = _bf16(T, Hq, D, seed=91), _bf16(T, Hkv, D, seed=92), _bf16(T, Hkv, D, seed=93)
    got = native.varlen_attention(q, k, v, lens, D ** -0.5)
    torch.cuda.synchronize()
    native.check_status()
    want = ref.varlen_attention(q.float(), k.float(), v.float(), lens, D ** -0.5)
    assert got.shape == q.shape
    _close(got, want, 2e-2, 2e-2)


def test_argmax_unaligned_rows(native):
    logits = torch.randn(7, 1003, device="cuda").to(torch.bfloat16)     # odd rows start off a 16-byte boundary
    assert torch.equal(native.argmax(logits).long(), torch.argmax(logits.float(), dim=-1))
    wide = torch.randn(5, 4099, device="cuda").to(torch.bfloat16)[:, :4096]   # aligned base, strided rows
    assert torch.equal(native.argmax(wide).long(), torch.argmax(wide.float(), dim=-1))


@pytest.mark.parametrize("P", [1, 16, 64])
@pytest.mark.parametrize("nq,tail", [(6, 6), (3, 9), (70, 70)])
def test_paged_extend_tail_mask(native, P, nq, tail):
    """Token-tree verification: the last `tail` keys follow an explicit mask, the prefix is visible."""
    Hq, Hkv, D = 8, 2, 128
    prefix = [0 + (tail - nq), 37 + (tail - nq), 128 + (tail - nq), 301 + (tail - nq)]
    B = len(prefix)
    seqs = [p + nq for p in prefix]
    cache, pt, rows = _attn_setup(B, seqs, P, Hkv, D, seed=40)
    q = _bf16(B * nq, Hq, D, seed=41)
    sl = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    pl = torch.tensor(prefix, dtype=torch.int32, device="cuda")
    cu = torch.arange(B + 1, dtype=torch.int32, device="cuda") * nq
    g = torch.Generator(device="cuda").manual_seed(42)
    mask = torch.rand(B, nq, tail, device="cuda", generator=g) < 0.5
    mask[:, :, 0] = True        # every row sees at least one tail key (sequence 0 may have no prefix)
    scale = D ** -0.5
    got = native.paged_attention(q, cache, pt, rows, sl, P, scale, cu, pl, tail_mask=mask)
    torch.cuda.synchronize()
    native.check_status()
    want = ref.paged_attention(q.float(), cache.float(), pt, rows, sl, P, scale, cu, pl, custom_mask=mask)
    _close(got, want, 2e-2, 2e-2)


def test_speculative_tree_kernels(native):
    from sglang_jax_b200.speculative import eagle_util
    g = torch.Generator().manual_seed(7)
    B, n, depth = 33, 12, 5
    # random trees: parent index < child index
    parent = torch.stack([torch.cat([torch.tensor([-1]), torch.stack([torch.randint(0, i, (1,), generator=g)[0]
                                                                      for i in range(1, n)])]) for _ in range(B)])
    tokens = torch.randint(0, 6, (B, n), generator=g)
    target = torch.randint(0, 6, (B, n), generator=g)
    acc_c, path_c, bonus_c = eagle_util.verify_tree_greedy(tokens, parent, target, depth)
    acc_g, path_g, bonus_g = native.verify_tree_greedy(tokens.cuda(), parent.cuda(), target.cuda(), depth)
    assert torch.equal(acc_g.cpu(), acc_c) and torch.equal(bonus_g.cpu(), bonus_c)
    assert torch.equal(path_g.cpu(), path_c)
    mask, dep = native.tree_mask(parent.cuda())
    for b in range(B):
        for i in range(n):
            anc, c = {i}, int(parent[b, i])
            while c >= 0:
                anc.add(c)
                c = int(parent[b, c])
            assert set(torch.nonzero(mask[b, i]).flatten().tolist()) == anc
            assert int(dep[b, i]) == len(anc) - 1


@pytest.mark.parametrize("T,K,outs,r", [(1, 1024, [512], 8), (37, 5120, [1024, 256, 256], 16), (300, 2048, [2048, 2048], 64)])
def test_lora_bgmv(native, T, K, outs, r):
    from sglang_jax_b200.lora.backend.base_backend import LoRABatchInfo
    from sglang_jax_b200.lora.backend.bgmv_backend import BgmvBackend
    slots = 4
    stack = len(outs)
    a = _bf16(slots, stack * r, K, scale=0.05, seed=50)
    bs = [_bf16(slots, n, r, scale=0.05, seed=51 + j) for j, n in enumerate(outs)]
    offs = [sum(outs[:j]) for j in range(stack)]
    x = _bf16(T, K, seed=60)
    y0 = _bf16(T, sum(outs), seed=61)
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(-1, slots, (T,), generator=g, dtype=torch.int32)
    scal = torch.tensor([0.5, 2.0, 1.0, 0.25], device="cuda")
    got = native.lora_bgmv(x, y0.clone(), a, bs, offs, tok.cuda(), scal)
    torch.cuda.synchronize()
    native.check_status()
    order = torch.argsort(tok, stable=True)
    st = tok[order]
    first = int((st < 0).sum())
    seg_slots, seg_bounds, i = [], [], first
    while i < T:
        j = i + int((st[i:] == st[i]).sum())
        seg_slots.append(int(st[i]))
        seg_bounds.append((i - first, j - first))
        i = j
    info = LoRABatchInfo(tok.cuda(), scal, None, True, order[first:].cuda(), seg_slots, seg_bounds)
    want = BgmvBackend._segments(x.float(), y0.float().clone(), a.float(), [b.float() for b in bs], offs, info)
    _close(got, want, 2e-2, 2e-2)


def test_kv_page_copy_device_host_roundtrip(native):
    """The page-copy kernel writes pinned host memory directly and reads it back (HiCache / PD staging)."""
    from sglang_jax_b200.mem_cache.host_kv_pool import LRUHostKVPool
    from sglang_jax_b200.mem_cache.memory_pool import MHATokenToKVPool
    pool = MHATokenToKVPool(64 * 16, 16, torch.bfloat16, 2, 128, 3, "cuda")
    for i, b in enumerate(pool.kv_buffer):
        b.copy_(_bf16(*b.shape, seed=70 + i))
    ref_bufs = [b.clone() for b in pool.kv_buffer]
    host = LRUHostKVPool(pool, 32)
    dev_pages = torch.tensor([3, 17, 40, 5, 64]).numpy()
    hp = host.alloc(5)
    host.backup_from_device(dev_pages, hp)
    torch.cuda.synchronize()
    for layer, b in enumerate(ref_bufs):
        assert torch.equal(host.host_views[layer][torch.as_tensor(hp)], b.view(b.shape[0], -1)[dev_pages].cpu())
    for b in pool.kv_buffer:
        b.zero_()
    new_pages = torch.tensor([9, 10, 11, 12, 13]).numpy()
    host.load_to_device(hp, new_pages)
    torch.cuda.synchronize()
    native.check_status()
    for layer, b in enumerate(ref_bufs):
        assert torch.equal(pool.kv_buffer[layer][new_pages], b[dev_pages])
        assert pool.kv_buffer[layer][20].abs().sum() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("P", [16, 64, 128])
@pytest.mark.parametrize("H", [16, 8, 40])
def test_mla_decode(native, P, H):
    """Absorbed-MLA decode kernel vs the fp32 PyTorch statement (ragged lengths, split-KV, head
    groups that are not full, page sizes below / at / above the tile)."""
    seqs = [1, 17, 64, 65, 300, 1000, 129, 1537]
    B = len(seqs)
    pages_per = [(s + P - 1) // P for s in seqs]
    num_pages = sum(pages_per) + 3
    g = torch.Generator(device="cuda").manual_seed(50)
    cache = (torch.randn(num_pages, P, 576, device="cuda", generator=g) * 0.5).bfloat16()
    pt = torch.zeros(B + 3, max(pages_per) + 2, dtype=torch.int32, device="cuda")
    perm = (torch.randperm(num_pages - 1, device="cuda") + 1).to(torch.int32)
    rows = torch.randperm(B + 2, device="cuda")[:B].to(torch.int32)
    o = 0
    for b in range(B):
        pt[rows[b], :pages_per[b]] = perm[o:o + pages_per[b]]
        o += pages_per[b]
    q_lat, q_pe = _bf16(B, H, 512, seed=51), _bf16(B, H, 64, seed=52)
    sl = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    scale = 192 ** -0.5
    expect = ref.mla_paged_attention(q_lat.float(), q_pe.float(), cache.float(), pt, rows, sl, P, scale, 512)
    assert native.mla_decode_supported(q_lat, q_pe, cache, 512, P)
    for splits in (1, 3, None):
        got = native.mla_decode(q_lat, q_pe, cache, pt, rows, sl, P, scale, max_seq_len=max(seqs), num_splits=splits)
        torch.cuda.synchronize()
        native.check_status()
        _close(got, expect, 2e-2, 2e-2)
    from sglang_jax_b200 import ops
    got = ops.mla_paged_attention(q_lat, q_pe, cache, pt, rows, sl, P, scale, 512, max_seq_len=max(seqs))
    _close(got, expect, 2e-2, 2e-2)


@pytest.mark.parametrize("Dk,Dv,H,Hqk,per_channel", [(128, 128, 8, 4, False), (64, 128, 4, 4, False), (128, 128, 4, 4, True),
                                                        (96, 64, 6, 2, True)])
def test_delta_rule_step_and_conv_update(native, Dk, Dv, H, Hqk, per_channel):
    """In-place recurrent decode kernels vs the fp32 PyTorch statements (GDN scalar gate with shared q/k
    heads, KDA per-channel gate), slots scattered through the pool, untouched slots left alone."""
    from sglang_jax_b200.ops import linear_attention as la
    B, n_slots = 5, 9
    g0 = torch.Generator(device="cuda").manual_seed(60)
    q, k, v = _bf16(B, Hqk, Dk, seed=61), _bf16(B, Hqk, Dk, seed=62), _bf16(B, H, Dv, seed=63)
    gate = -torch.rand((B, H, Dk) if per_channel else (B, H), device="cuda", generator=g0)
    beta = torch.rand(B, H, device="cuda", generator=g0)
    pool = torch.randn(n_slots, H, Dk, Dv, device="cuda", generator=g0) * 0.1
    slots = torch.tensor([7, 2, 5, 1, 8], device="cuda")
    before = pool.clone()
    r = H // Hqk
    qe, ke = q.repeat_interleave(r, 1), k.repeat_interleave(r, 1)
    if per_channel:
        want_o, want_S = la.kda_recurrent(qe[:, None], ke[:, None], v[:, None], gate[:, None], beta[:, None], before[slots])
        want_o = want_o[:, 0]
    else:
        want_o, want_S = la.recurrent_gated_delta_rule_step(qe, ke, v, gate, beta, before[slots])
    got = native.delta_rule_step(q, k, v, gate, beta, pool, slots, gate_per_channel=per_channel)
    torch.cuda.synchronize()
    _close(got, want_o, 2e-2, 2e-2)
    assert torch.allclose(pool[slots], want_S, atol=2e-3, rtol=2e-3)
    rest = [i for i in range(n_slots) if i not in slots.tolist()]
    assert torch.equal(pool[rest], before[rest])
    # short convolution
    C, K = 3 * Hqk * Dk, 4
    x, w = _bf16(B, C, seed=64), _bf16(C, K, seed=65)
    for dt in (torch.bfloat16, torch.float32):
        cpool = (torch.randn(n_slots, C, K - 1, device="cuda", generator=g0)).to(dt)
        cb = cpool.clone()
        want_y, want_state = la.causal_conv1d_update(x, cb[slots], w)
        y = native.conv1d_update(x, cpool, w, slots)
        torch.cuda.synchronize()
        _close(y, want_y, 2e-2, 2e-2)
        assert torch.allclose(cpool[slots].float(), want_state.to(dt).float(), atol=1e-2)
        assert torch.equal(cpool[rest], cb[rest])


@pytest.mark.parametrize("M,N,K", [(128, 1024, 512), (5, 256, 4096), (300, 384, 1040), (1, 5120, 5120), (1024, 2048, 2048)])
def test_gemm_fp8_per_token_per_channel(native, M, N, K):
    """e4m3 x e4m3 tcgen05 GEMM with per-token / per-channel scales vs the fp32 product of the same
    quantised operands (decode and prefill tilings, ragged M, K not a multiple of the 128-byte block)."""
    from sglang_jax_b200.utils.quantization import quantize_activation, quantize_tensor
    g = torch.Generator(device="cuda").manual_seed(70)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    bias = _bf16(N, seed=71)
    xq, xs = quantize_activation(x, torch.float8_e4m3fn)
    wq, ws = quantize_tensor(w, torch.float8_e4m3fn, "per_channel")
    want = (xq.float() @ wq.float().t()) * xs * ws.t() + bias.float()
    got = native.gemm_fp8(xq, wq.contiguous(), xs, ws, bias)
    torch.cuda.synchronize()
    native.check_status()
    _close(got, want, 2e-2, 2e-2)
    full = x @ w.t() + bias.float()
    assert ((got.float() - full).norm() / full.norm()).item() < 0.08       # and close to the unquantised product


# ------------------------------------------------------------------------------------------
# The tensor-parallel kernels with world == 1 (loop-back on one GPU): the same code paths as on 2..8
# GPUs (peer stores land in this GPU's own buffers, flag waits are met by the launch itself).
def _fused_case(T, H, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(T, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(H, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    res = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    nw = (torch.randn(H, device="cuda", generator=g) * 0.1 + 1).to(torch.bfloat16)
    y = (x.float() @ w.float().t()).to(torch.bfloat16).float() + res.float()
    new_res = y.to(torch.bfloat16)
    return x, w, res, nw, new_res, ref.rmsnorm(new_res, nw, 1e-6)


@pytest.mark.parametrize("T", [1, 7, 128, 200, 300, 1100])
@pytest.mark.parametrize("defer", [False, True])
def test_fused_gemm_rs_norm_ag_loopback(native, T, defer):
    from sglang_jax_b200.parallel.fused_comm import FusedComm
    H, K, N2 = 1024, 512, 768
    comm = FusedComm.create_loopback(H, "cuda", max_tokens=2048)
    for it in range(3):      # repeated launches reuse buffers, flags and counters
        x, w, res, nw, want_res, want = _fused_case(T, H, K, 100 + it)
        got_res = res.clone()
        out, _ = comm.gemm_allreduce_add_rmsnorm(x, w, got_res, nw, 1e-6, defer=defer)
        if defer:
            g = torch.Generator(device="cuda").manual_seed(7 + it)
            w2 = (torch.randn(N2, H, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
            y2 = comm.consume_linear(out, w2)
            assert comm.pending_gather is None
            want2 = (want.float() @ w2.float().t())
            err2 = (y2.float() - want2).abs().max().item()
            assert err2 < 0.06 * max(1.0, want2.abs().max().item()), (T, it, err2)
        torch.cuda.synchronize()
        native.check_status()
        err = (out.float() - want.float()).abs().max().item()
        rerr = (got_res.float() - want_res.float()).abs().max().item()
        assert err < 0.1 and rerr < 0.07, (T, it, err, rerr)
    assert int(comm.fseq.item()) == 3 and int(comm.fctrs.abs().sum().item()) == 0


def test_fused_two_kernel_path_and_gathers_loopback(native):
    """The GEMM-with-push-epilogue + reduce kernel pair, the cross-rank argmax and the logits gather at world == 1."""
    from sglang_jax_b200.parallel.fused_comm import FusedComm
    H, K = 1024, 512
    comm = FusedComm.create_loopback(H, "cuda", max_tokens=1024)
    comm.one_kernel = False
    for T in (5, 128, 400):
        x, w, res, nw, want_res, want = _fused_case(T, H, K, 200 + T)
        got_res = res.clone()
        out, _ = comm.gemm_allreduce_add_rmsnorm(x, w, got_res, nw, 1e-6)
        torch.cuda.synchronize()
        native.check_status()
        assert (out.float() - want.float()).abs().max().item() < 0.1
        assert (got_res.float() - want_res.float()).abs().max().item() < 0.07
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(37, 1000, device="cuda", generator=g)
    logits[3, 10] = logits[3, 700] = 50.0
    ids = comm.argmax_gather(logits, 0, 995)
    assert ids.long().tolist() == torch.argmax(logits[:, :995], dim=-1).tolist()
    lb = logits.to(torch.bfloat16)
    assert torch.equal(comm.logits_gather(lb), lb)
    torch.cuda.synchronize()
    native.check_status()


# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (100, 384, 1024), (128, 7168, 2048), (300, 2048, 7168), (1000, 1536, 512)])
def test_gemm_fp8_block_scaled(native, M, N, K):
    """128 x 128 block-scaled weights x per-token-group-128 activations against the fp32 product of the very
    same quantised operands."""
    from sglang_jax_b200.utils.quantization import dequantize_tensor, quantize_tensor
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = (torch.randn(M, K, device="cuda", generator=g) * torch.rand(M, 1, device="cuda", generator=g) * 3).to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    w[: N // 2] *= 7.0                     # very different block magnitudes
    wq, sw = quantize_tensor(w, torch.float8_e4m3fn, "block", (128, 128))
    xq, sx = native.quant_fp8_group128(x)
    assert native.gemm_fp8_block_supported(wq, sw, (128, 128))
    # the quantiser: scales are amax / 448 per (token, 128 group) and the values round-trip
    xg = x.float().view(M, K // 128, 128)
    want_s = (xg.abs().amax(-1) / 448.0).clamp_min(1e-12).t()
    assert torch.allclose(sx[:, :M], want_s, rtol=1e-5, atol=0)
    xd = (xq.float().view(M, K // 128, 128) * sx[:, :M].t()[..., None]).view(M, K)
    assert (xd - x.float()).abs().max() <= 0.07 * x.float().abs().max()
    y = native.gemm_fp8_block(xq, sx, wq, sw)
    want = xd @ dequantize_tensor(wq, sw, (128, 128), torch.float32).t()
    torch.cuda.synchronize()
    native.check_status()
    _close(y, want, atol=0.02 * want.abs().max().item(), rtol=0.02)


@pytest.mark.parametrize("T,E,E_local,e0,k,H,I", [(5, 8, 8, 0, 2, 256, 128), (128, 16, 4, 8, 4, 512, 256),
                                                  (700, 8, 8, 0, 2, 1024, 384)])
def test_fused_experts_fp8_block_scaled(native, T, E, E_local, e0, k, H, I):
    """Expert FFN on 128 x 128 block-scaled e4m3 weights with per-token-group-128 activation scales (grouped
    block-scaled tcgen05 GEMM) vs the PyTorch statement on the same quantised weights."""
    from sglang_jax_b200.layers.moe import FusedMoE, _fp8_reference_experts
    moe = FusedMoE(E, H, I, tp_size=E // E_local, tp_rank=e0 // E_local, ep_size=E // E_local).cuda()
    moe.w13_weight.data.copy_(_bf16(E_local, 2 * I, H, scale=0.05, seed=61))
    moe.w2_weight.data.copy_(_bf16(E_local, H, I, scale=0.05, seed=62))
    x = _bf16(T, H, seed=60)
    logits = torch.randn(T, E, device="cuda", generator=torch.Generator(device="cuda").manual_seed(63))
    tw, ids = ref.topk_route(logits, k)
    full = ref.moe_forward(x.float(), moe.w13_weight.float(), moe.w2_weight.float(), tw, ids, e0)
    moe.quantize_(torch.float8_e4m3fn, (128, 128), torch.float8_e4m3fn)
    assert moe.fp8_block and moe.w13_weight.dtype == torch.float8_e4m3fn
    assert moe.w13_scale.shape == (E_local, 2 * I // 128, H // 128) and moe.w2_scale.shape == (E_local, H // 128, I // 128)
    got = moe(x, tw, ids)
    torch.cuda.synchronize()
    native.check_status()
    want = _fp8_reference_experts(x, moe, tw, ids)
    assert ((got.float() - want.float()).norm() / want.float().norm()).item() < 0.03
    assert ((got.float() - full).norm() / full.norm()).item() < 0.1


@pytest.mark.parametrize("P", [16, 64, 128])
def test_paged_extend_tcgen05_long_and_rescaled(native, P):
    """The tcgen05 prefill kernel (head_dim 128): long sequences over many 128-key tiles, prefixes that are not
    tile aligned, and scores that grow along the sequence so that the running maximum is raised (and the
    accumulator in tensor memory rescaled) many times."""
    Hq, Hkv, D = 8, 2, 128
    prefix = [0, 300, 1000, 7]
    ext = [700, 129, 1, 2048]
    seqs = [a + b for a, b in zip(prefix, ext)]
    B = len(seqs)
    cache, pt, rows = _attn_setup(B, seqs, P, Hkv, D, seed=70)
    T = sum(ext)
    q = _bf16(T, Hq, D, seed=71)
    # keys later in a page get larger norms: maxima keep growing along a sequence
    ramp = torch.linspace(0.2, 3.0, P, device="cuda").view(1, 1, P, 1)
    cache[:, 0] = (cache[:, 0].float() * ramp).to(torch.bfloat16)
    sl = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    pl = torch.tensor(prefix, dtype=torch.int32, device="cuda")
    cu = torch.zeros(B + 1, dtype=torch.int32, device="cuda")
    cu[1:] = torch.tensor(ext, device="cuda").cumsum(0)
    for scale in (D ** -0.5, 0.6):
        got = native.paged_attention(q, cache, pt, rows, sl, P, scale, cu, pl)
        torch.cuda.synchronize()
        native.check_status()
        _close(got, ref.paged_attention(q.float(), cache.float(), pt, rows, sl, P, scale, cu, pl), 3e-2, 3e-2)


@pytest.mark.parametrize("M,N,K", [(128, 1280, 5120), (128, 6400, 5120), (128, 5120, 3200), (16, 51200, 5120),
                                   (1, 10240, 5120), (100, 5120, 1024), (7, 1000, 640), (33, 256, 64)])
def test_gemm_decode_cluster_split_k(native, M, N, K):
    """Split-K inside thread-block clusters with the reduction through distributed shared memory vs the fp32 product
    (cluster sizes 1..8, ragged M, N not a multiple of the tile, ranks with unequal K ranges, bias)."""
    x = _bf16(M, K, seed=90)
    w = (_bf16(N, K, seed=91).float() * 0.05).bfloat16()
    bias = _bf16(N, seed=92)
    cs = native.lib().sglb_gemm_decode_cluster_size(M, N, K)
    assert cs in (1, 2, 4, 8)
    for b in (None, bias):
        got = native.gemm_decode_cluster(x, w, b)
        again = native.gemm_decode_cluster(x, w, b)
        torch.cuda.synchronize()
        native.check_status()
        want = x.float() @ w.float().t() + (b.float() if b is not None else 0.0)
        _close(got, want, 2e-2, 2e-2)
        assert torch.equal(got, again)                    # fixed summation order: bitwise repeatable
    # out-of-range shapes are refused, not run
    assert native.lib().sglb_gemm_decode_cluster_size(129, N, K) == 0
    assert native.lib().sglb_gemm_decode_cluster_size(M, N, K + 8) == 0
