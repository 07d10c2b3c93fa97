"""ctypes bindings of `libsglb200.so` (the sm_100a kernels under `csrc/`).

The library has a plain C ABI: raw device pointers, sizes and a `cudaStream_t`.  Tensors
are passed by `data_ptr()`, outputs are allocated here with torch (which also makes them
CUDA-graph capturable), and every launch goes to torch's current stream.  A non-zero
return code raises; `check_status()` reads the device status word that bounded waits
write when they give up.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_size_t, c_void_p

import torch

_LIB = None
# SGLB_BOUNDS_CHECK=1: the checked build of the library (see csrc/build.py)
_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)),
                         "libsglb200_checked.so" if os.environ.get("SGLB_BOUNDS_CHECK", "0") == "1"
                         else "libsglb200.so")
LOADED = False


def lib():
    global _LIB, LOADED
    if _LIB is not None:
        return _LIB
    if not os.path.exists(_LIB_PATH):
        # source checkout on a box with nvcc: build on first use
        try:
            from ..csrc.build import build
            build()
        except Exception as e:
            raise RuntimeError(
                f"native kernel library {_LIB_PATH} is missing and could not be built ({e}); "
                f"run `python -m sglang_jax_b200.csrc.build`") from e
    L = ctypes.CDLL(_LIB_PATH)
    L.sglb_version.restype = ctypes.c_char_p
    L.sglb_gemm_decode_cluster.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    L.sglb_gemm_decode_cluster_size.argtypes = [c_int, c_int, c_int]
    L.sglb_enable_peer_access.argtypes = [c_int, c_int]
    if hasattr(L, "sglb_debug_set_kv_pages"):
        L.sglb_debug_set_kv_pages.argtypes = [c_int]
    L.sglb_gemm_workspace_bytes.restype = c_size_t
    L.sglb_gemm_workspace_bytes.argtypes = [c_int, c_int, c_int]
    L.sglb_gemm_max_counters.argtypes = [c_int]
    L.sglb_gemm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t,
                                 c_void_p, c_int, c_int, c_void_p]
    L.sglb_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_float, c_int, c_void_p]
    L.sglb_fused_add_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_float, c_int,
                                         c_void_p]
    L.sglb_silu_and_mul.argtypes = [c_void_p, c_void_p, c_longlong, c_int, c_void_p]
    L.sglb_embedding.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p]
    L.sglb_argmax.argtypes = [c_void_p, c_void_p, c_int, c_int, c_longlong, c_int, c_void_p]
    L.sglb_rope_qknorm_kvwrite.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                           c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                           c_void_p]
    L.sglb_page_table_scatter.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
    L.sglb_resolve_future.argtypes = [c_void_p, c_void_p, c_int, c_void_p]
    L.sglb_decode_num_splits.argtypes = [c_int, c_int, c_int]
    L.sglb_gemm_fp8.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                c_size_t, c_void_p, c_void_p]
    L.sglb_sample_filtered.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
    L.sglb_quant_fp8_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p]
    L.sglb_delta_rule_step.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    L.sglb_conv1d_update.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                     c_void_p]
    L.sglb_mla_decode.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
                                  c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p]
    L.sglb_paged_decode.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_float, c_int, c_void_p,
                                    c_void_p, c_void_p]
    L.sglb_paged_extend.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                    c_float, c_void_p]
    L.sglb_paged_extend_masked.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_float, c_int, c_float, c_void_p, c_int, c_int, c_void_p]
    L.sglb_verify_tree_greedy.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                          c_int, c_void_p]
    L.sglb_tree_mask.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
    L.sglb_lora_shrink.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    L.sglb_lora_expand.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_void_p]
    L.sglb_kv_page_copy.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_longlong,
                                    c_longlong, c_void_p]
    L.sglb_read_status.argtypes = [c_void_p]
    _LIB = L
    LOADED = True
    return L


# number of kernel launches issued through this module (bench bookkeeping)
launch_count = 0


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Raw handle of the current CUDA stream (the private getter skips building a Stream object per launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str):
    global launch_count
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"native op {what} failed with code {rc}")


def _p(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def check_status():
    """Raise if a kernel recorded a bounded-wait timeout (synchronises the device)."""
    buf = (c_int * 4)()
    code = lib().sglb_read_status(buf)
    if code != 0:
        names = {1: "timeout waiting for TMA data", 2: "timeout waiting for a free stage",
                 3: "timeout waiting for the accumulator", 4: "timeout waiting for TMEM to drain",
                 5: "timeout waiting for a peer flag", 6: "bad argument",
                 7: "index out of bounds (checked build; the access was skipped)"}
        raise RuntimeError(f"kernel status {code} ({names.get(code, '?')}), block={buf[1]} aux=({buf[2]}, {buf[3]})")


# ------------------------------------------------------------------------------------ ops
def rmsnorm(x, w, eps, gemma=False):
    x = x.contiguous()
    y = torch.empty_like(x)
    H = x.shape[-1]
    _check(lib().sglb_rmsnorm(_p(y), _p(x), _p(w), x.numel() // H, H, eps, int(gemma), _stream()), "rmsnorm")
    return y


def fused_add_rmsnorm(x, residual, w, eps, gemma=False):
    """Updates `residual` in place; returns (normed, residual)."""
    x = x.contiguous()
    assert residual.is_contiguous()
    y = torch.empty_like(x)
    H = x.shape[-1]
    _check(lib().sglb_fused_add_rmsnorm(_p(y), _p(x), _p(residual), _p(w), x.numel() // H, H, eps, int(gemma),
                                        _stream()), "fused_add_rmsnorm")
    return y, residual


def silu_and_mul(x):
    x = x.contiguous()
    I = x.shape[-1] // 2
    out = torch.empty((*x.shape[:-1], I), dtype=x.dtype, device=x.device)
    _check(lib().sglb_silu_and_mul(_p(out), _p(x), x.numel() // (2 * I), I, _stream()), "silu_and_mul")
    return out


class _GemmScratch:
    """Per-device split-K workspace (fp32 partial tiles) and tile counters.  Allocated once,
    outside any CUDA-graph capture, and shared by every GEMM on the stream (launches on one
    stream are ordered, and the kernel leaves the counters zeroed)."""

    def __init__(self, device):
        self.bytes = 128 << 20
        self.workspace = torch.empty(self.bytes, dtype=torch.uint8, device=device)
        self.counters = torch.zeros(4096, dtype=torch.int32, device=device)


_scratch: dict = {}


def gemm_scratch(device) -> _GemmScratch:
    key = (device.type, device.index)
    s = _scratch.get(key)
    if s is None:
        s = _GemmScratch(device)
        _scratch[key] = s
    return s


# measured plan of decode-sized GEMM shapes (model_executor/tuning_cache.GemmPlan), set by the model runner
gemm_plan = None
LIBRARY_GEMM = 2          # plan entry: the library GEMM measured faster than both operand assignments for this shape
CLUSTER_GEMM = 3          # plan entry: split-K inside thread-block clusters (csrc/gemm_decode_cluster.cu)
_PLAN_CLUSTER = os.environ.get("SGLB_GEMM_PLAN_CLUSTER", "1") == "1"


def gemm_decode_cluster(x2, w, bias=None, out=None):
    """`x2 [M <= 128, K] @ w [N, K]^T (+ bias)` with the cluster split-K kernel; K a multiple of 64, N of 8."""
    M, K = x2.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=x2.dtype, device=x2.device)
    L = lib()
    _check(L.sglb_gemm_decode_cluster(_p(x2), _p(w), _p(bias), _p(out), M, N, K, _stream()), "gemm_decode_cluster")
    return out


def _library_gemm(x2, w, bias, out):
    if bias is None:
        torch.matmul(x2, w.t(), out=out)
    else:
        torch.addmm(bias, x2, w.t(), out=out)


def linear(x, w, bias=None, force_mode: int = -1, force_splits: int = 0, out=None):
    K = x.shape[-1]
    N = w.shape[0]
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M = x2.shape[0]
    if K % 8 or N % 8 or not w.is_contiguous() or x2.data_ptr() % 16 or w.data_ptr() % 16:
        from . import reference
        y = reference.linear(x, w, bias)
        if out is not None:
            out.copy_(y.view_as(out))
            return out
        return y
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    else:
        assert out.is_contiguous() and out.numel() == M * N and out.data_ptr() % 16 == 0
        out = out.view(M, N)
    if M == 0:
        return out.view(*x.shape[:-1], N)
    sc = gemm_scratch(x.device)
    if gemm_plan is not None and force_mode < 0 and M <= 256:
        def run(mode):
            if mode == LIBRARY_GEMM:
                _library_gemm(x2, w, bias, out)
            elif mode == CLUSTER_GEMM:
                lib().sglb_gemm_decode_cluster(_p(x2), _p(w), _p(bias), _p(out), M, N, K, _stream())
            else:
                lib().sglb_gemm_bf16(_p(x2), _p(w), _p(bias), _p(out), M, N, K, _p(sc.workspace), sc.bytes,
                                     _p(sc.counters), mode, 0, _stream())
        cluster_ok = (_PLAN_CLUSTER and M <= 128 and K % 64 == 0
                      and lib().sglb_gemm_decode_cluster_size(M, N, K) > 0)
        force_mode = gemm_plan.mode_for(M, N, K, run, extra=(CLUSTER_GEMM,) if cluster_ok else ())
        if force_mode == LIBRARY_GEMM:
            _library_gemm(x2, w, bias, out)
            return out.view(*x.shape[:-1], N)
        if force_mode == CLUSTER_GEMM:
            if cluster_ok:
                gemm_decode_cluster(x2, w, bias, out)
                return out.view(*x.shape[:-1], N)
            force_mode = -1          # a table entry measured for another M of the same bucket
    _check(lib().sglb_gemm_bf16(_p(x2), _p(w), _p(bias), _p(out), M, N, K, _p(sc.workspace), sc.bytes,
                                _p(sc.counters), force_mode, force_splits, _stream()), "gemm_bf16")
    return out.view(*x.shape[:-1], N)


def rope_qknorm_kvwrite(qkv, positions, cos_sin, q_norm_w, k_norm_w, eps, num_q_heads, num_kv_heads, head_dim,
                        kv_buffer, out_cache_loc, page_size, is_neox=True, rotary_dim=None):
    qkv = qkv.contiguous()
    T = qkv.shape[0]
    rd = rotary_dim or head_dim
    if (is_neox and cos_sin is not None and (rd // 2) % 32 != 0) or head_dim not in (64, 128, 256) \
            or positions.dtype != torch.int32 or (out_cache_loc is not None and out_cache_loc.dtype != torch.int32):
        from . import reference
        return reference.rope_qknorm_kvwrite(qkv, positions, cos_sin, q_norm_w, k_norm_w, eps, num_q_heads,
                                             num_kv_heads, head_dim, kv_buffer, out_cache_loc, page_size, is_neox,
                                             rotary_dim)
    q = torch.empty((T, num_q_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    _check(lib().sglb_rope_qknorm_kvwrite(_p(q), _p(qkv), _p(positions), _p(cos_sin), _p(q_norm_w), _p(k_norm_w),
                                          eps, T, num_q_heads, num_kv_heads, head_dim, rd, _p(kv_buffer),
                                          _p(out_cache_loc), page_size, int(is_neox), _stream()),
           "rope_qknorm_kvwrite")
    return q


def decode_num_splits(B: int, Hkv: int, max_seq_len: int) -> int:
    return lib().sglb_decode_num_splits(B, Hkv, max(max_seq_len, 1))


# SGLB_EXTEND_TC=0 keeps prefill attention on the mma.sync kernel (A/B switch)
_EXTEND_TC = os.environ.get("SGLB_EXTEND_TC", "1") != "0"


def paged_attention(q, kv_buffer, page_table, req_pool_indices, seq_lens, page_size, scale, cu_q_lens=None,
                    prefix_lens=None, sliding_window=0, soft_cap=0.0, max_q_len=0, max_seq_len=0, num_splits=None,
                    tail_mask=None):
    T, Hq, D = q.shape
    Hkv = kv_buffer.shape[2]
    B = req_pool_indices.shape[0]
    ok_page = (64 % page_size == 0) if page_size < 64 else (page_size % 64 == 0)
    if not ok_page or Hq // Hkv > 16:
        from . import reference
        return reference.paged_attention(q, kv_buffer, page_table, req_pool_indices, seq_lens, page_size, scale,
                                         cu_q_lens, prefix_lens, sliding_window, soft_cap, None, tail_mask)
    q = q.contiguous()
    out = torch.empty_like(q)
    num_pages = kv_buffer.shape[0]
    max_pages = page_table.shape[1]
    L = lib()
    if cu_q_lens is None:
        if num_splits is None:
            num_splits = decode_num_splits(B, Hkv, max_seq_len or page_table.shape[1] * page_size)
        part_o = part_lse = None
        if num_splits > 1:
            part_o = torch.empty((B, Hq, num_splits, D), dtype=torch.float32, device=q.device)
            part_lse = torch.empty((B, Hq, num_splits), dtype=torch.float32, device=q.device)
        _check(L.sglb_paged_decode(_p(q), _p(out), _p(kv_buffer), num_pages, _p(page_table), max_pages,
                                   _p(req_pool_indices), _p(seq_lens), B, Hq, Hkv, D, page_size, scale,
                                   int(sliding_window or 0), float(soft_cap or 0.0), num_splits, _p(part_o),
                                   _p(part_lse), _stream()), "paged_decode")
    elif tail_mask is not None:
        # [B, rows, tail] visibility of the trailing keys (speculative trees / bidirectional blocks)
        tm = tail_mask.to(torch.uint8).contiguous()
        bound = T // 64 + B
        _check(L.sglb_paged_extend_masked(_p(q), _p(out), _p(kv_buffer), num_pages, _p(page_table), max_pages,
                                          _p(req_pool_indices), _p(seq_lens), _p(prefix_lens), _p(cu_q_lens), B,
                                          bound, Hq, Hkv, D, page_size, scale, int(sliding_window or 0),
                                          float(soft_cap or 0.0), _p(tm), tm.shape[2], tm.shape[1], _stream()),
               "paged_extend_masked")
    elif D == 128 and not sliding_window and not soft_cap and _EXTEND_TC:
        # causal prefill on the tcgen05 kernel: 128-row query tiles, S and O in tensor memory
        L.sglb_paged_extend_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_int, c_float, c_int, c_void_p]
        _check(L.sglb_paged_extend_tc(_p(q), _p(out), _p(kv_buffer), num_pages, _p(page_table), max_pages,
                                      _p(req_pool_indices), _p(seq_lens), _p(prefix_lens), _p(cu_q_lens), B,
                                      T // 128 + B, T, Hq, Hkv, D, page_size, scale, 0, _stream()), "paged_extend_tc")
    else:
        bound = T // 64 + B
        _check(L.sglb_paged_extend(_p(q), _p(out), _p(kv_buffer), num_pages, _p(page_table), max_pages,
                                   _p(req_pool_indices), _p(seq_lens), _p(prefix_lens), _p(cu_q_lens), B, bound, Hq,
                                   Hkv, D, page_size, scale, int(sliding_window or 0), float(soft_cap or 0.0),
                                   _stream()), "paged_extend")
    return out


def pack_varlen_pages(k, v, lens, page_size: int = 64):
    """`k, v [T, H, D]` of sequences with lengths `lens`, packed along T -> a paged cache
    `[pages, 2, H, page_size, D]` in which every sequence starts on a page boundary (page 0 is an all-zero dummy),
    its page table `[B, max_pages]`, `lens` and their running sum as int32 device tensors, and the two counts."""
    T, H, D = k.shape
    dev, P, B = k.device, page_size, len(lens)
    pages = [(n + P - 1) // P for n in lens]
    max_pages = max(max(pages, default=0), 1)
    base, table = 1, []
    for np_ in pages:
        table.append([base + i for i in range(np_)] + [0] * (max_pages - np_))
        base += np_
    i32 = dict(dtype=torch.int32, device=dev)
    lens_t = torch.tensor(lens, **i32)
    cu = torch.zeros(B + 1, **i32)
    cu[1:] = torch.cumsum(lens_t, 0)
    pos = torch.arange(T, device=dev) - torch.repeat_interleave(cu[:-1].long(), lens_t.long())
    first_page = torch.tensor([row[0] for row in table], device=dev, dtype=torch.long)
    page_of = torch.repeat_interleave(first_page, lens_t.long()) + pos // P
    cache = torch.zeros((base, 2, H, P, D), dtype=k.dtype, device=dev)
    cache[page_of, 0, :, pos % P] = k
    cache[page_of, 1, :, pos % P] = v
    return cache, torch.tensor(table, **i32), lens_t, cu, base, max_pages


def varlen_attention(q, k, v, seq_lens, scale: float):
    """Bidirectional attention over a ragged batch of sequences packed along the token axis (vision / audio
    encoders, diffusion transformers): `q [T, Hq, D]`, `k, v [T, Hkv, D]`, `seq_lens` host ints summing to T.
    K / V are laid out as 64-token pages (one gather-friendly copy) and the paged extend kernel runs with the
    causal rule switched off; head dims that are not 64 / 128 are zero-padded to the next of the two
    (reference kernel: `python/sgl_jax/srt/multimodal/kernels/varlen_attention.py`)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    lens = [int(x) for x in seq_lens]
    assert sum(lens) == T and q.dtype == torch.bfloat16 and Hq % Hkv == 0 and Hq // Hkv <= 16 and D <= 128
    Dp = 64 if D <= 64 else 128
    if Dp != D:
        pad = lambda t: torch.nn.functional.pad(t, (0, Dp - D))
        q, k, v = pad(q), pad(k), pad(v)
    P, B = 64, len(lens)
    cache, pt, lens_t, cu, base, max_pages = pack_varlen_pages(k, v, lens, P)
    i32 = dict(dtype=torch.int32, device=q.device)
    rows = torch.arange(B, **i32)
    prefix = torch.zeros(B, **i32)
    qc = q.contiguous()
    out = torch.empty_like(qc)
    _check(lib().sglb_paged_extend_masked(_p(qc), _p(out), _p(cache), base, _p(pt), max_pages, _p(rows), _p(lens_t),
                                          _p(prefix), _p(cu), B, T // 64 + B, Hq, Hkv, Dp, P,
                                          float(scale), 0, 0.0, None, 0, -1, _stream()), "varlen_attention")
    return out[..., :D] if Dp != D else out


def sample_filtered(logits, temperatures, top_ks, top_ps, min_ps, seeds, positions, return_probs: bool = False,
                    request_seeded: bool = True):
    """Temperature / top-k / top-p / min-p filtering and hashed Gumbel-max sampling of `logits [B, V]` (fp32 or
    bf16, unit stride inside a row) in one kernel -> int32 `[B]` ids (and, with `return_probs`, the filtered
    renormalised fp32 probabilities).  `request_seeded` keeps the reference's (seed, position, column) hash bit
    for bit; without it the uniforms come from an avalanche mix of the same inputs."""
    assert logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)
    B, V = logits.shape
    dev = logits.device
    f32 = lambda t: t.to(device=dev, dtype=torch.float32).reshape(-1).contiguous()
    i32 = lambda t: t.to(device=dev, dtype=torch.int32).reshape(-1).contiguous()
    temperatures, top_ps, min_ps = f32(temperatures), f32(top_ps), f32(min_ps)
    top_ks, seeds, positions = i32(top_ks.clamp(max=2 ** 31 - 1)), i32(seeds), i32(positions)
    for t in (temperatures, top_ps, min_ps, top_ks, seeds, positions):
        assert t.numel() == B
    out = torch.empty(B, dtype=torch.int32, device=dev)
    probs = torch.empty((B, V), dtype=torch.float32, device=dev) if return_probs else None
    _check(lib().sglb_sample_filtered(_p(out), _p(probs), _p(logits), B, V, logits.stride(0), logits.element_size(),
                                      _p(temperatures), _p(top_ks), _p(top_ps), _p(min_ps), _p(seeds), _p(positions),
                                      0 if request_seeded else 1, _stream()), "sample_filtered")
    return (out, probs) if return_probs else out


def quant_fp8_rows(x, gated: bool = False, valid_rows=None):
    """Per-token dynamic e4m3 quantisation of `x [T, K]` bf16 -> `(q [T, K], scale [T])`.  `gated`: `x` is
    `[T, 2K]` and `silu(x[:, :K]) * x[:, K:]` is quantised.  `valid_rows`: device int32 scalar; rows at or
    past it are skipped (their outputs stay uninitialised)."""
    assert x.dtype == torch.bfloat16
    x = x.contiguous()
    K = x.shape[-1] // (2 if gated else 1)
    T = x.numel() // x.shape[-1]
    q = torch.empty((*x.shape[:-1], K), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    _check(lib().sglb_quant_fp8_rows(_p(q), _p(s), _p(x), T, K, int(gated),
                                     valid_rows.data_ptr() if valid_rows is not None else None, _stream()),
           "quant_fp8_rows")
    return q, s


def quant_fp8_group128(x, valid_rows=None):
    """Per-token-group (1 x 128) dynamic e4m3 quantisation of `x [T, K]` bf16 (K a multiple of 128) ->
    `(q [T, K], scale [K / 128, T])`: the activation format of 128 x 128 block-scaled weights."""
    assert x.dtype == torch.bfloat16 and x.shape[-1] % 128 == 0
    x = x.contiguous()
    K = x.shape[-1]
    T = x.numel() // K
    q = torch.empty((T, K), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((K // 128, max(T, 1)), dtype=torch.float32, device=x.device)
    L = lib()
    L.sglb_quant_fp8_group128.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
    _check(L.sglb_quant_fp8_group128(_p(x), _p(q), _p(s), T, K, max(T, 1),
                                     valid_rows.data_ptr() if valid_rows is not None else None, _stream()),
           "quant_fp8_group128")
    return q, s


def gemm_fp8_block_supported(wq, scale_w, block_size) -> bool:
    return (wq.dtype == torch.float8_e4m3fn and tuple(block_size or ()) == (128, 128) and wq.dim() == 2
            and wq.shape[1] % 128 == 0 and wq.shape[0] % 8 == 0 and wq.is_contiguous() and wq.data_ptr() % 16 == 0
            and tuple(scale_w.shape) == ((wq.shape[0] + 127) // 128, wq.shape[1] // 128))


def gemm_fp8_block(xq, sx, wq, sw, bias=None):
    """Block-scaled e4m3 product (DeepSeek-V3 format): `xq [M, K]` with group scales `sx [K/128, >=M]`, `wq [N, K]`
    with block scales `sw [ceil(N/128), K/128]` -> bf16 `[M, N]`; every 128-wide K block is promoted with its two
    scales into fp32 accumulators (`csrc/gemm_fp8_block.cu`)."""
    M, K = xq.shape
    N = wq.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=xq.device)
    if M == 0:
        return out
    L = lib()
    L.sglb_gemm_fp8_block.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                      c_int, c_void_p]
    sw = sw.float().contiguous()
    _check(L.sglb_gemm_fp8_block(_p(xq), _p(wq), _p(sx), sx.shape[1], _p(sw), _p(bias), _p(out), M, N, K, _stream()),
           "gemm_fp8_block")
    return out


def gemm_fp8_supported(xq, wq) -> bool:
    return (xq.dtype == torch.float8_e4m3fn and wq.dtype == torch.float8_e4m3fn and xq.shape[-1] % 16 == 0
            and wq.shape[0] % 8 == 0 and wq.is_contiguous() and wq.data_ptr() % 16 == 0)


def gemm_fp8(xq, wq, scale_x, scale_w, bias=None, out_dtype=torch.bfloat16):
    """`(xq [M, K] . wq [N, K]^T) * scale_x [M] * scale_w [N] + bias` with e4m3 operands on the tcgen05
    `kind::f8f6f4` path (fp32 accumulation), bf16 result."""
    assert out_dtype == torch.bfloat16
    K, N = xq.shape[-1], wq.shape[0]
    x2 = xq.reshape(-1, K).contiguous()
    M = x2.shape[0]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=xq.device)
    if M == 0:
        return out.view(*xq.shape[:-1], N)
    sx = scale_x.reshape(-1).float().contiguous()
    sw = scale_w.reshape(-1).float().contiguous()
    assert sx.numel() == M and sw.numel() == N
    sc = gemm_scratch(xq.device)
    _check(lib().sglb_gemm_fp8(_p(x2), _p(wq), _p(sx), _p(sw), _p(bias), _p(out), M, N, K, _p(sc.workspace), sc.bytes,
                               _p(sc.counters), _stream()), "gemm_fp8")
    return out.view(*xq.shape[:-1], N)


def delta_rule_step(q, k, v, g, beta, state_pool, slots, gate_per_channel=False, l2norm=True):
    """One recurrent step per request, state updated in place.  `q, k [B, Hqk, Dk]`, `v [B, H, Dv]` bf16,
    `g [B, H]` (or `[B, H, Dk]`) and `beta [B, H]` fp32, `state_pool [slots, H, Dk, Dv]` fp32,
    `slots [B]` int64 -> `o [B, H, Dv]` bf16."""
    B, H, Dv = v.shape
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    g, beta = g.float().contiguous(), beta.float().contiguous()
    assert state_pool.dtype == torch.float32 and state_pool.is_contiguous() and slots.dtype == torch.int64
    out = torch.empty_like(v)
    _check(lib().sglb_delta_rule_step(_p(q), _p(k), _p(v), _p(g), _p(beta), _p(state_pool), _p(slots), _p(out), B, H,
                                      q.shape[1], q.shape[2], Dv, int(gate_per_channel), int(l2norm), _stream()),
           "delta_rule_step")
    return out


def conv1d_update(x, state_pool, weight, slots, silu=True):
    """Short causal convolution of one new input per request; `state_pool [slots, C, K-1]` (bf16 or fp32)
    is shifted in place.  `x [B, C]` bf16, `weight [C, K]` bf16 -> `y [B, C]` bf16."""
    B, C = x.shape
    x, weight = x.contiguous(), weight.contiguous()
    assert state_pool.is_contiguous() and state_pool.dtype in (torch.bfloat16, torch.float32) and slots.dtype == torch.int64
    y = torch.empty_like(x)
    _check(lib().sglb_conv1d_update(_p(x), _p(state_pool), _p(weight), _p(slots), _p(y), B, C, weight.shape[1],
                                    int(silu), int(state_pool.dtype == torch.bfloat16), _stream()), "conv1d_update")
    return y


def mla_decode_supported(q_latent, q_pe, kv_buffer, kv_lora_rank, page_size) -> bool:
    return (q_latent.dtype == torch.bfloat16 and kv_buffer.dtype == torch.bfloat16 and kv_lora_rank == 512
            and q_pe.shape[-1] == 64 and kv_buffer.shape[-1] == 576
            and ((64 % page_size == 0) if page_size < 64 else (page_size % 64 == 0)))


def mla_decode(q_latent, q_pe, kv_buffer, page_table, req_pool_indices, seq_lens, page_size, scale, max_seq_len=0,
               num_splits=None):
    """Absorbed-MLA decode: `q_latent [B, H, 512]`, `q_pe [B, H, 64]`, latent cache
    `[pages, P, 576]` -> latent output `[B, H, 512]` (the caller applies W_UV)."""
    B, H, R = q_latent.shape
    q_latent, q_pe = q_latent.contiguous(), q_pe.contiguous()
    out = torch.empty_like(q_latent)
    if num_splits is None:
        num_splits = decode_num_splits(B, (H + 15) // 16, max_seq_len or page_table.shape[1] * page_size)
    part_o = part_lse = None
    if num_splits > 1:
        part_o = torch.empty((B, H, num_splits, R), dtype=torch.float32, device=q_latent.device)
        part_lse = torch.empty((B, H, num_splits), dtype=torch.float32, device=q_latent.device)
    _check(lib().sglb_mla_decode(_p(q_latent), _p(q_pe), _p(out), _p(kv_buffer), kv_buffer.shape[0], _p(page_table),
                                 page_table.shape[1], _p(req_pool_indices), _p(seq_lens), B, H, R, q_pe.shape[-1],
                                 page_size, scale, num_splits, _p(part_o), _p(part_lse), _stream()), "mla_decode")
    return out


def lora_bgmv(x, y, a_buf, b_bufs, out_offsets, token_slots, scalings):
    """`y[:, off_j:off_j+N_j] += scale[slot] * B_j[slot] (A[slot] x)[j*r:(j+1)*r]` per token, in place.
    `a_buf [slots, stack*r, K]`, `b_bufs[j] [slots, N_j, r]`, `token_slots [T]` int32 (-1 = skip)."""
    T, K = x.shape
    R = a_buf.shape[1]
    r = R // len(b_bufs)
    x = x.contiguous()
    assert y.stride(-1) == 1
    h = torch.empty((T, R), dtype=torch.float32, device=x.device)
    L = lib()
    _check(L.sglb_lora_shrink(_p(h), _p(x), _p(a_buf), _p(token_slots), T, R, K, _stream()), "lora_shrink")
    for j, (b, off) in enumerate(zip(b_bufs, out_offsets)):
        _check(L.sglb_lora_expand(_p(y), _p(h), _p(b), _p(token_slots), _p(scalings), T, b.shape[1], r, R, j * r,
                                  y.stride(0), int(off), _stream()), "lora_expand")
    return y


def kv_page_copy(dst: torch.Tensor, src: torch.Tensor, dst_pages: torch.Tensor, src_pages: torch.Tensor):
    """`dst[dst_pages[i]] = src[src_pages[i]]` for 2-D page tables `[pages, page_elems]`; either tensor may
    be pinned host memory.  Index tensors are int64 on the device.  Asynchronous on the current stream."""
    n = dst_pages.numel()
    if n == 0:
        return
    assert dst.dim() == 2 and src.dim() == 2 and dst.shape[1] == src.shape[1] and dst.dtype == src.dtype
    assert dst.stride(1) == 1 and src.stride(1) == 1
    es = dst.element_size()
    _check(lib().sglb_kv_page_copy(dst.data_ptr(), src.data_ptr(), _p(dst_pages), _p(src_pages), n,
                                   dst.shape[1] * es, dst.stride(0) * es, src.stride(0) * es, _stream()),
           "kv_page_copy")


def set_debug_kv_pages(pages: int) -> bool:
    """Checked build (`SGLB_BOUNDS_CHECK=1`): give the KV-write kernel the extent of the KV buffers; a slot outside
    them is then reported by `check_status()` and its store skipped.  False when the loaded library has no checks."""
    L = lib()
    if not hasattr(L, "sglb_debug_set_kv_pages"):
        return False
    rc = L.sglb_debug_set_kv_pages(int(pages))
    if rc < 0:
        raise RuntimeError(f"sglb_debug_set_kv_pages failed with code {rc}")
    return rc == 1


def enable_peer_access(device: torch.device, peer: torch.device) -> None:
    """Allow kernels on `device` to read / write memory of `peer` (both CUDA devices of this process)."""
    if device.index == peer.index:
        return
    rc = lib().sglb_enable_peer_access(int(device.index), int(peer.index))
    if rc < 0:
        raise RuntimeError(f"cuda:{device.index} cannot access the memory of cuda:{peer.index} (no peer path)")
    _check(rc, "enable_peer_access")


def verify_tree_greedy(tokens, parent, target_ids, max_depth: int):
    """`(accept [B], path [B, max_depth+1], bonus [B])`, all int64; see `speculative/eagle_util.py`."""
    B, n = tokens.shape
    tok = tokens.long().contiguous()
    par = parent.long().contiguous()
    tgt = target_ids.long().contiguous()
    accept = torch.empty(B, dtype=torch.long, device=tok.device)
    path = torch.empty((B, max_depth + 1), dtype=torch.long, device=tok.device)
    bonus = torch.empty(B, dtype=torch.long, device=tok.device)
    _check(lib().sglb_verify_tree_greedy(_p(tok), _p(par), _p(tgt), _p(accept), _p(path), _p(bonus), B, n,
                                         int(max_depth), _stream()), "verify_tree_greedy")
    return accept, path, bonus


def tree_mask(parent):
    """Ancestor mask `[B, n, n]` (uint8) and depths `[B, n]` of trees given by parent indices."""
    B, n = parent.shape
    par = parent.long().contiguous()
    mask = torch.empty((B, n, n), dtype=torch.uint8, device=par.device)
    depth = torch.empty((B, n), dtype=torch.long, device=par.device)
    _check(lib().sglb_tree_mask(_p(par), _p(mask), _p(depth), B, n, _stream()), "tree_mask")
    return mask, depth


def embedding(ids, table, vocab_start=0, masked=False):
    ids = ids.contiguous()
    T = ids.numel()
    H = table.shape[1]
    out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    _check(lib().sglb_embedding(_p(out), _p(ids), _p(table), T, H, table.shape[0], vocab_start, int(masked),
                                _stream()), "embedding")
    return out.view(*ids.shape, H)


def argmax(logits):
    assert logits.dim() == 2 and logits.stride(1) == 1
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _check(lib().sglb_argmax(_p(out), _p(logits), B, V, logits.stride(0), logits.element_size(), _stream()),
           "argmax")
    return out


def page_table_scatter(table, rows, pos, ids):
    n = rows.numel()
    _check(lib().sglb_page_table_scatter(_p(table), table.shape[1], _p(rows), _p(pos), _p(ids), n, _stream()),
           "page_table_scatter")


def resolve_future(ids, future_map):
    _check(lib().sglb_resolve_future(_p(ids), _p(future_map), ids.numel(), _stream()), "resolve_future")
    return ids
