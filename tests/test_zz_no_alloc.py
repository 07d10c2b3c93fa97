"""Allocation-free GEMM entry point.

Some embedders of this library may not allocate device memory once they are running: an
engine that has already handed nearly all of HBM to its weight arena and KV pool (a late
cudaMalloc can fail or stall the device), or a plugin inside a host runtime that owns all
device allocations.  For them `sglb_gemm_bf16_noalloc` keeps its split-K scratch in a static
device array inside the library.  This test calls it through its exported C symbol and checks
it against the regular entry point (`sglb_gemm_bf16`, reached through `native.linear`) on two
consecutive calls that share that scratch.  It is collected last so that a run that stops at
the first failure has already exercised everything else.
"""

import ctypes
from ctypes import c_int, c_size_t, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from sglang_jax_b200.ops import native
    L = native.lib()
    L.sglb_gemm_bf16_noalloc.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    L.sglb_gemm_bf16_noalloc.restype = c_int
    L.sglb_gemm_bf16_noalloc_scratch_bytes.restype = c_size_t
    L.sglb_gemm_bf16_noalloc_last_error.restype = ctypes.c_char_p
    L.sglb_gemm_bf16_noalloc_status.argtypes = [c_void_p]
    return L, native


def _call(L, x, w, b, out, splits):
    M, K = x.shape
    N = w.shape[0]
    return L.sglb_gemm_bf16_noalloc(x.data_ptr(), w.data_ptr(), b.data_ptr() if b is not None else None,
                                    out.data_ptr(), M, N, K, splits, torch.cuda.current_stream().cuda_stream)


def test_noalloc_gemm_matches_regular_entry_point():
    L, native = _lib()
    assert L.sglb_gemm_bf16_noalloc_scratch_bytes() == (8 << 20) + 8192
    g = torch.Generator(device="cuda").manual_seed(123)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)

    # two calls in a row, different shapes and split counts, same static scratch
    cases = [(96, 1024, 4096, 4, True), (17, 2048, 2048, 0, False)]
    for M, N, K, splits, with_bias in cases:
        x, w = rnd(M, K), rnd(N, K, scale=0.05)
        b = rnd(N) if with_bias else None
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        rc = _call(L, x, w, b, out, splits)
        assert rc == 0, L.sglb_gemm_bf16_noalloc_last_error()
        expect = native.linear(x, w, b)
        torch.cuda.synchronize()
        st = (c_int * 4)()
        assert L.sglb_gemm_bf16_noalloc_status(st) == 0, list(st)
        ref32 = x.float() @ w.float().t() + (b.float() if b is not None else 0)
        err = (out.float() - expect.float()).abs()
        tol = 2e-2 + 1.5e-2 * ref32.abs()
        assert (err > tol).float().mean().item() < 1e-4, f"max err {err.max().item()}"
        assert ((out.float() - ref32).abs() > 0.1 + 1.5e-2 * ref32.abs()).float().mean().item() < 1e-4


def test_noalloc_gemm_rejects_oversize():
    L, _ = _lib()
    x = torch.zeros(300, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(300, 64, device="cuda", dtype=torch.bfloat16)
    assert _call(L, x, w, None, out, 0) < 0
    assert b"256" in L.sglb_gemm_bf16_noalloc_last_error()
    # 16 splits of 400 tiles x 128 x 256 fp32 do not fit in 8 MiB
    x = torch.zeros(256, 8192, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(51200, 8192, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(256, 51200, device="cuda", dtype=torch.bfloat16)
    assert _call(L, x, w, None, out, 16) < 0
    assert b"scratch" in L.sglb_gemm_bf16_noalloc_last_error()
