#!/usr/bin/env python
"""Kernel micro-benchmarks with roofline fractions (counterpart of the reference's
`benchmark/kernels/*`): CUDA-event timing after warm-up, L2 flushed between iterations,
achieved TFLOP/s or GB/s and the fraction of the measured peaks in MEASURED_PEAKS.json.

    python benchmark/kernels/bench_kernels.py gemm attention elementwise moe sampling
"""

from __future__ import annotations

import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from sglang_jax_b200.ops import native  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def timeit(fn, iters=20, warmup=3, flush=True):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            _flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm():
    hbm, tf, src = peaks()
    shapes = [  # (M, N, K, label)  Qwen3-32B TP1 and TP8 shards
        (8192, 10240, 5120, "qkv prefill tp1"), (8192, 5120, 8192, "o prefill tp1"),
        (8192, 51200, 5120, "gate_up prefill tp1"), (8192, 5120, 25600, "down prefill tp1"),
        (8192, 6400, 5120, "gate_up prefill tp8"), (8192, 5120, 3200, "down prefill tp8"),
        (4096, 10240, 5120, "qkv prefill 4k"), (1024, 5120, 5120, "mid"),
        (128, 10240, 5120, "qkv decode tp1"), (128, 5120, 8192, "o decode tp1"),
        (128, 51200, 5120, "gate_up decode tp1"), (128, 5120, 25600, "down decode tp1"),
        (128, 1280, 5120, "qkv decode tp8"), (128, 6400, 5120, "gate_up decode tp8"),
        (128, 5120, 3200, "down decode tp8"), (128, 18992, 5120, "lm_head decode tp8"),
        (16, 51200, 5120, "gate_up bs16"), (1, 51200, 5120, "gate_up bs1"),
    ]
    print(f"{'shape':>28} {'label':>22} {'ours ms':>9} {'TFLOP/s':>9} {'GB/s':>8} {'roof%':>7} {'torch ms':>9} {'vs torch':>8} {'cluster ms':>10}")
    native.gemm_plan = None            # the persistent kernel with its own default choice, not the measured plan
    for M, N, K, label in shapes:
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        t = timeit(lambda: native.linear(x, w))
        tt = timeit(lambda: torch.nn.functional.linear(x, w))
        tc = None
        if M <= 128 and K % 64 == 0 and native.lib().sglb_gemm_decode_cluster_size(M, N, K) > 0:
            o = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            tc = timeit(lambda: native.gemm_decode_cluster(x, w, None, o))
        flops = 2.0 * M * N * K
        byts = 2.0 * (M * K + N * K + M * N)
        tfl = flops / t / 1e9
        gbs = byts / t / 1e6
        roof = max(flops / (tf * 1e12), byts / (hbm * 1e9)) * 1e3   # ms at the roofline
        print(f"{f'{M}x{N}x{K}':>28} {label:>22} {t:9.4f} {tfl:9.1f} {gbs:8.0f} {100 * roof / t:6.1f}% {tt:9.4f} {tt / t:8.2f} "
              + (f"{tc:10.4f}" if tc is not None else f"{'-':>10}"))
    print(f"{'fp8 e4m3 (per-token x per-channel scales)':>51} {'fp8 ms':>9} {'TFLOP/s':>9} {'GB/s':>8} {'bf16 ms':>9}")
    for M, N, K, label in [(8192, 10240, 5120, "qkv prefill tp1"), (8192, 51200, 5120, "gate_up prefill tp1"),
                           (128, 10240, 5120, "qkv decode tp1"), (128, 51200, 5120, "gate_up decode tp1"),
                           (128, 5120, 25600, "down decode tp1"), (16, 51200, 5120, "gate_up bs16")]:
        xq = torch.randn(M, K, device="cuda").to(torch.float8_e4m3fn)
        wq = (torch.randn(N, K, device="cuda") * 0.5).to(torch.float8_e4m3fn)
        sx, sw = torch.rand(M, device="cuda") + 0.5, torch.rand(N, device="cuda") + 0.5
        x, w = xq.to(torch.bfloat16), wq.to(torch.bfloat16)
        t = timeit(lambda: native.gemm_fp8(xq, wq, sx, sw))
        tb = timeit(lambda: native.linear(x, w))
        byts = 1.0 * (M * K + N * K) + 2.0 * M * N
        print(f"{f'{M}x{N}x{K}':>28} {label:>22} {t:9.4f} {2.0 * M * N * K / t / 1e9:9.1f} {byts / t / 1e6:8.0f} {tb:9.4f}")
    print(f"{'fp8 e4m3 (1x128 activation groups, 128x128 weight blocks)':>51} {'fp8 ms':>9} {'TFLOP/s':>9} {'GB/s':>8} {'quant ms':>9}")
    for M, N, K, label in [(8192, 7168, 2048, "deepseek o_proj"), (8192, 4096, 7168, "deepseek up"),
                           (4096, 10240, 5120, "qkv prefill 4k"), (128, 7168, 18432, "deepseek down decode"),
                           (128, 51200, 5120, "gate_up decode tp1")]:
        x = torch.randn(M, K, device="cuda").bfloat16()
        wq = (torch.randn(N, K, device="cuda") * 0.5).to(torch.float8_e4m3fn)
        sw = torch.rand((N + 127) // 128, K // 128, device="cuda") + 0.5
        xq, sx = native.quant_fp8_group128(x)
        t = timeit(lambda: native.gemm_fp8_block(xq, sx, wq, sw))
        tq = timeit(lambda: native.quant_fp8_group128(x))
        byts = 1.0 * (M * K + N * K) + 2.0 * M * N
        print(f"{f'{M}x{N}x{K}':>28} {label:>22} {t:9.4f} {2.0 * M * N * K / t / 1e9:9.1f} {byts / t / 1e6:8.0f} {tq:9.4f}")
    torch.cuda.synchronize()
    native.check_status()
    print(f"(roofline = slower of FLOPs / {tf} TFLOP/s and bytes / {hbm} GB/s, {src})")


def bench_attention():
    hbm, tf, src = peaks()
    print(f"{'case':>40} {'ms':>9} {'GB/s':>8} {'of hbm':>7}")
    D, P = 128, 64
    for B, Hq, Hkv, S in [(128, 64, 8, 1400), (128, 32, 4, 1400), (128, 16, 2, 1400), (128, 8, 1, 1400), (128, 64, 8, 2300),
                          (32, 64, 8, 4096), (256, 8, 1, 1400), (16, 64, 8, 1400)]:
        pages_per = (S + P - 1) // P
        num_pages = B * pages_per + 1
        cache = torch.randn(num_pages, 2, Hkv, P, D, device="cuda").bfloat16()
        pt = (torch.arange(B * pages_per, device="cuda", dtype=torch.int32) + 1).view(B, pages_per).contiguous()
        rows = torch.arange(B, device="cuda", dtype=torch.int32)
        sl = torch.full((B,), S, device="cuda", dtype=torch.int32)
        q = torch.randn(B, Hq, D, device="cuda").bfloat16()
        t = timeit(lambda: native.paged_attention(q, cache, pt, rows, sl, P, D ** -0.5, max_seq_len=S))
        byts = B * S * 2 * Hkv * D * 2
        print(f"{f'decode B={B} Hq={Hq} Hkv={Hkv} S={S}':>40} {t:9.4f} {byts / t / 1e6:8.0f} {100 * byts / t / 1e6 / hbm:6.1f}%")
    for B, H, S in [(128, 16, 1400), (128, 128, 1400), (32, 16, 8192), (256, 16, 1400)]:   # absorbed MLA (latent 512 + 64)
        pages_per = (S + P - 1) // P
        cache = torch.randn(B * pages_per + 1, P, 576, device="cuda").bfloat16()
        pt = (torch.arange(B * pages_per, device="cuda", dtype=torch.int32) + 1).view(B, pages_per).contiguous()
        rows = torch.arange(B, device="cuda", dtype=torch.int32)
        sl = torch.full((B,), S, device="cuda", dtype=torch.int32)
        ql, qp = torch.randn(B, H, 512, device="cuda").bfloat16(), torch.randn(B, H, 64, device="cuda").bfloat16()
        t = timeit(lambda: native.mla_decode(ql, qp, cache, pt, rows, sl, P, 192 ** -0.5, max_seq_len=S))
        byts = B * S * 576 * 2
        print(f"{f'mla decode B={B} H={H} S={S}':>40} {t:9.4f} {byts / t / 1e6:8.0f} {100 * byts / t / 1e6 / hbm:6.1f}%")
    print(f"{'case':>40} {'ms':>9} {'TFLOP/s':>8}")
    for B, Hq, Hkv, S in [(4, 64, 8, 2048), (8, 8, 1, 1024), (1, 64, 8, 8192)]:
        pages_per = (S + P - 1) // P
        num_pages = B * pages_per + 1
        cache = torch.randn(num_pages, 2, Hkv, P, D, device="cuda").bfloat16()
        pt = (torch.arange(B * pages_per, device="cuda", dtype=torch.int32) + 1).view(B, pages_per).contiguous()
        rows = torch.arange(B, device="cuda", dtype=torch.int32)
        sl = torch.full((B,), S, device="cuda", dtype=torch.int32)
        pl = torch.zeros(B, device="cuda", dtype=torch.int32)
        cu = (torch.arange(B + 1, device="cuda", dtype=torch.int32) * S).contiguous()
        q = torch.randn(B * S, Hq, D, device="cuda").bfloat16()
        t = timeit(lambda: native.paged_attention(q, cache, pt, rows, sl, P, D ** -0.5, cu, pl), iters=5)
        flops = 4.0 * B * Hq * D * S * S / 2
        print(f"{f'extend B={B} Hq={Hq} Hkv={Hkv} S={S}':>40} {t:9.4f} {flops / t / 1e9:8.1f}")
    torch.cuda.synchronize()
    native.check_status()


def bench_moe():
    """Routed-expert FFN (align, gather, two grouped GEMMs, activation, combine): bf16 vs W8A8 e4m3."""
    from sglang_jax_b200.layers.moe import FusedMoE
    from sglang_jax_b200.ops import reference
    hbm, tf, src = peaks()
    print(f"{'case':>44} {'bf16 ms':>9} {'fp8 ms':>9} {'bf16 TFLOP/s':>13} {'fp8 TFLOP/s':>12} {'fp8 GB/s':>9}")
    for T, E, k, H, I, label in [(128, 128, 8, 2048, 768, "qwen3-30b-a3b decode"), (8192, 128, 8, 2048, 768, "qwen3-30b-a3b prefill"),
                                 (128, 32, 8, 7168, 2048, "deepseek-v3 ep8 decode"), (8192, 32, 8, 7168, 2048, "deepseek-v3 ep8 prefill")]:
        moe = FusedMoE(E, H, I, tp_size=1, tp_rank=0, ep_size=1).cuda()
        moe.w13_weight.data.normal_(0, 0.02)
        moe.w2_weight.data.normal_(0, 0.02)
        x = torch.randn(T, H, device="cuda").bfloat16()
        tw, ids = reference.topk_route(torch.randn(T, E, device="cuda"), k)
        ids = ids.int()
        tb = timeit(lambda: moe(x, tw, ids))
        moe.quantize_(torch.float8_e4m3fn, None, torch.float8_e4m3fn)
        t8 = timeit(lambda: moe(x, tw, ids))
        flops = 2.0 * T * k * 3 * I * H
        touched = min(E, T * k)
        byts = touched * 3.0 * I * H
        print(f"{f'T={T} E={E} k={k} H={H} I={I} {label}':>44} {tb:9.4f} {t8:9.4f} {flops / tb / 1e9:13.1f} {flops / t8 / 1e9:12.1f} {byts / t8 / 1e6:9.0f}")
        del moe
    torch.cuda.synchronize()
    native.check_status()


def bench_sampling():
    """Filtered sampling at the Qwen3 vocabulary: one radix-select kernel vs the sort-based PyTorch statement."""
    from sglang_jax_b200.ops import reference
    print(f"{'case':>44} {'kernel ms':>10} {'torch ms':>9}")
    V = 151936
    for B, k, p, mp, label in [(128, 50, 0.95, 0.0, "top-k 50 top-p .95"), (128, V, 0.9, 0.0, "top-p .9"),
                               (128, V, 1.0, 0.0, "temperature only"), (128, 20, 1.0, 0.05, "top-k 20 min-p .05"),
                               (16, 50, 0.95, 0.0, "top-k 50 top-p .95")]:
        logits = torch.randn(B, V, device="cuda") * 2
        one = lambda v, dt=torch.float32: torch.full((B,), v, device="cuda", dtype=dt)
        t, ks, ps, mps = one(0.7), one(k, torch.int32), one(p), one(mp)
        seeds, pos = torch.arange(B, device="cuda", dtype=torch.int32), torch.arange(B, device="cuda", dtype=torch.int32)
        tk = timeit(lambda: native.sample_filtered(logits, t, ks, ps, mps, seeds, pos), flush=False)
        tt = timeit(lambda: reference.multinomial_with_seed(
            reference.top_k_top_p_min_p_probs(logits, t, ks.long(), ps, mps), seeds, pos), iters=5, flush=False)
        print(f"{f'B={B} V={V} {label}':>44} {tk:10.4f} {tt:9.4f}")
    torch.cuda.synchronize()
    native.check_status()


def bench_elementwise():
    hbm, tf, src = peaks()
    T, H, I = 8192, 5120, 25600
    x = torch.randn(T, H, device="cuda").bfloat16()
    r = torch.randn(T, H, device="cuda").bfloat16()
    w = torch.ones(H, device="cuda").bfloat16()
    t = timeit(lambda: native.fused_add_rmsnorm(x, r, w, 1e-6))
    print(f"fused_add_rmsnorm {T}x{H}: {t:.4f} ms, {4 * T * H * 2 / t / 1e6:.0f} GB/s ({100 * 4 * T * H * 2 / t / 1e6 / hbm:.1f}% of {src} copy bw)")
    g = torch.randn(T, 2 * I // 8, device="cuda").bfloat16()
    t = timeit(lambda: native.silu_and_mul(g))
    print(f"silu_and_mul {T}x{I // 8}: {t:.4f} ms, {3 * T * (I // 8) * 2 / t / 1e6:.0f} GB/s")


if __name__ == "__main__":
    which = sys.argv[1:] or ["gemm", "attention", "elementwise"]
    torch.manual_seed(0)
    for w in which:
        {"gemm": bench_gemm, "attention": bench_attention, "elementwise": bench_elementwise, "moe": bench_moe, "sampling": bench_sampling}[w]()
