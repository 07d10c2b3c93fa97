#!/usr/bin/env python
"""One small, self-terminating case per kernel for `ncu` captures (inputs larger than L2, a few
hundred MB on the device, a handful of launches).

    python benchmark/kernels/profile_case.py gemm_prefill|gemm_decode|attn_decode|attn_extend|sampling|gemm_fp8|gemm_fp8_block|moe_fp8|decode_step:<architecture>
"""

import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from sglang_jax_b200.ops import native  # noqa: E402


def main():
    case = sys.argv[1]
    n = int(sys.argv[2]) if len(sys.argv) > 2 else 4
    torch.manual_seed(0)
    if case in ("gemm_prefill", "gemm_decode"):
        M, N, K = (4096, 5120, 5120) if case == "gemm_prefill" else (128, 51200, 5120)
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        for _ in range(n):
            native.linear(x, w)
    elif case == "attn_decode":
        B, Hq, Hkv, S, D, P = 128, 64, 8, 1400, 128, 64
        pp = (S + P - 1) // P
        cache = torch.randn(B * pp + 1, 2, Hkv, P, D, device="cuda").bfloat16()
        pt = (torch.arange(B * pp, device="cuda", dtype=torch.int32) + 1).view(B, pp).contiguous()
        rows = torch.arange(B, device="cuda", dtype=torch.int32)
        sl = torch.full((B,), S, device="cuda", dtype=torch.int32)
        q = torch.randn(B, Hq, D, device="cuda").bfloat16()
        for _ in range(n):
            native.paged_attention(q, cache, pt, rows, sl, P, D ** -0.5, max_seq_len=S)
    elif case == "attn_extend":
        B, Hq, Hkv, S, D, P = 4, 64, 8, 2048, 128, 64
        pp = (S + P - 1) // P
        cache = torch.randn(B * pp + 1, 2, Hkv, P, D, device="cuda").bfloat16()
        pt = (torch.arange(B * pp, device="cuda", dtype=torch.int32) + 1).view(B, pp).contiguous()
        rows = torch.arange(B, device="cuda", dtype=torch.int32)
        sl = torch.full((B,), S, device="cuda", dtype=torch.int32)
        pl = torch.zeros(B, device="cuda", dtype=torch.int32)
        cu = (torch.arange(B + 1, device="cuda", dtype=torch.int32) * S).contiguous()
        q = torch.randn(B * S, Hq, D, device="cuda").bfloat16()
        for _ in range(n):
            native.paged_attention(q, cache, pt, rows, sl, P, D ** -0.5, cu, pl)
    elif case == "sampling":
        B, V = 256, 151936                                   # 155 MB of fp32 logits: larger than L2
        logits = torch.randn(B, V, device="cuda") * 2
        one = lambda v, dt=torch.float32: torch.full((B,), v, device="cuda", dtype=dt)
        seeds = torch.arange(B, device="cuda", dtype=torch.int32)
        for _ in range(n):
            native.sample_filtered(logits, one(0.7), one(50, torch.int32), one(0.95), one(0.0), seeds, seeds)
    elif case == "gemm_fp8":
        M, N, K = 4096, 10240, 5120
        xq = torch.randn(M, K, device="cuda").to(torch.float8_e4m3fn)
        wq = (torch.randn(N, K, device="cuda") * 0.5).to(torch.float8_e4m3fn)
        sx, sw = torch.rand(M, device="cuda") + 0.5, torch.rand(N, device="cuda") + 0.5
        for _ in range(n):
            native.gemm_fp8(xq, wq, sx, sw)
    elif case == "gemm_fp8_block":
        M, N, K = 4096, 7168, 4096
        x = torch.randn(M, K, device="cuda").bfloat16()
        wq = (torch.randn(N, K, device="cuda") * 0.5).to(torch.float8_e4m3fn)
        sw = torch.rand((N + 127) // 128, K // 128, device="cuda") + 0.5
        for _ in range(n):
            xq, sx = native.quant_fp8_group128(x)
            native.gemm_fp8_block(xq, sx, wq, sw)
    elif case == "moe_fp8":
        from sglang_jax_b200.layers.moe import FusedMoE
        from sglang_jax_b200.ops import reference
        T, E, k, H, I = 2048, 32, 8, 7168, 2048
        moe = FusedMoE(E, H, I, tp_size=1, tp_rank=0, ep_size=1).cuda()
        moe.w13_weight.data.normal_(0, 0.02)
        moe.w2_weight.data.normal_(0, 0.02)
        moe.quantize_(torch.float8_e4m3fn, None, torch.float8_e4m3fn)
        x = torch.randn(T, H, device="cuda").bfloat16()
        tw, ids = reference.topk_route(torch.randn(T, E, device="cuda"), k)
        ids = ids.int()
        for _ in range(n):
            moe(x, tw, ids)
    elif case.startswith("decode_step:"):
        # whole decode steps of a named architecture with random weights straight on the model runner (captured CUDA
        # graph replays): `decode_step:qwen3-32b-tp8-shard [steps] [batch] [context]`; meant for a launch list
        import tempfile
        from sglang_jax_b200.bench_one_batch import run_one_batch
        from sglang_jax_b200.server_args import ServerArgs
        from sglang_jax_b200.utils.tiny_models import ARCH_CONFIGS, write_config_only
        B = int(sys.argv[3]) if len(sys.argv) > 3 else 128
        ctx = int(sys.argv[4]) if len(sys.argv) > 4 else 1024
        path = write_config_only(tempfile.mkdtemp(prefix="sglb_case_"), dict(ARCH_CONFIGS[case.split(":", 1)[1]]))
        sa = ServerArgs(model_path=path, load_format="dummy", device="cuda", dtype="bfloat16", page_size=64,
                        skip_tokenizer_init=True, max_running_requests=B, cuda_graph_max_bs=B,
                        max_total_tokens=(B + 2) * (ctx + 64 * 3), mem_fraction_static=0.8, log_level="error",
                        chunked_prefill_size=-1, max_prefill_tokens=B * ctx + 64)
        print(run_one_batch(sa, B, ctx, n))
    else:
        raise SystemExit(f"unknown case {case}")
    torch.cuda.synchronize()
    native.check_status()
    print("ok", case)


if __name__ == "__main__":
    main()
