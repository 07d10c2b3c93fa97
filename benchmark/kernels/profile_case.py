#!/usr/bin/env python
"""One small, self-terminating case per kernel for `ncu` captures (inputs larger than L2, a few
hundred MB on the device, a handful of launches).

    python benchmark/kernels/profile_case.py gemm_prefill|gemm_decode|attn_decode|attn_extend|ar_norm
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
    else:
        raise SystemExit(f"unknown case {case}")
    torch.cuda.synchronize()
    native.check_status()
    print("ok", case)


if __name__ == "__main__":
    main()
