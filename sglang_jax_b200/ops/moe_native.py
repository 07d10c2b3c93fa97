"""ctypes bindings of the MoE kernels (`csrc/moe.cu`, grouped GEMM in `csrc/gemm_sm100.cu`)."""

from __future__ import annotations

from ctypes import c_float, c_int, c_size_t, c_void_p

import torch

from . import native

_bound = False


def _lib():
    global _bound
    L = native.lib()
    if not _bound:
        L.sglb_topk_route.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                      c_int, c_int, c_float, c_void_p]
        L.sglb_moe_align.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p]
        L.sglb_moe_gather.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        L.sglb_moe_combine.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
        L.sglb_grouped_gemm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_int, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]
        L.sglb_grouped_gemm_fp8.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_size_t,
                                            c_void_p, c_void_p]
        _bound = True
    return L


_SCORING = {"softmax": 0, "sigmoid": 1, "tanh": 2}


def topk_route(router_logits, top_k, scoring="softmax", renormalize=True, correction_bias=None,
               num_expert_group=0, topk_group=0, routed_scaling_factor=1.0):
    T, E = router_logits.shape
    router_logits = router_logits.contiguous()
    w = torch.empty((T, top_k), dtype=torch.float32, device=router_logits.device)
    ids = torch.empty((T, top_k), dtype=torch.int32, device=router_logits.device)
    bias = correction_bias.float().contiguous() if correction_bias is not None else None
    rc = _lib().sglb_topk_route(router_logits.data_ptr(), router_logits.element_size(),
                                bias.data_ptr() if bias is not None else None, w.data_ptr(), ids.data_ptr(), T, E,
                                top_k, _SCORING[scoring], int(renormalize), int(num_expert_group or 0),
                                int(topk_group or 0), float(routed_scaling_factor), native._stream())
    native._check(rc, "topk_route")
    return w, ids


class MoeWorkspace:
    """Index buffers of one MoE layer call, sized for `max_pairs` routed (token, expert) pairs."""

    def __init__(self, max_pairs: int, num_local_experts: int, device):
        self.max_pairs = max_pairs
        i32 = dict(dtype=torch.int32, device=device)
        self.offsets = torch.zeros(num_local_experts + 1, **i32)
        self.pair_row = torch.empty(max_pairs, **i32)
        self.row_token = torch.empty(max_pairs, **i32)
        self.tile_group = torch.empty(max_pairs // 128 + num_local_experts + 1, **i32)
        self.tile_row0 = torch.empty(max_pairs // 128 + num_local_experts + 1, **i32)
        self.counts = torch.zeros(2, **i32)


def moe_align(topk_ids, expert_start, num_local_experts, ws: MoeWorkspace, expert_hist=None):
    T, k = topk_ids.shape
    rc = _lib().sglb_moe_align(topk_ids.data_ptr(), T * k, k, expert_start, num_local_experts, ws.offsets.data_ptr(),
                               ws.pair_row.data_ptr(), ws.row_token.data_ptr(), ws.tile_group.data_ptr(),
                               ws.tile_row0.data_ptr(), ws.counts.data_ptr(),
                               expert_hist.data_ptr() if expert_hist is not None else None, native._stream())
    native._check(rc, "moe_align")


def moe_gather(x, ws: MoeWorkspace, max_rows: int):
    H = x.shape[-1]
    out = torch.empty((max_rows, H), dtype=x.dtype, device=x.device)
    rc = _lib().sglb_moe_gather(out.data_ptr(), x.data_ptr(), ws.row_token.data_ptr(), ws.counts.data_ptr(),
                                max_rows, H, native._stream())
    native._check(rc, "moe_gather")
    return out


def grouped_gemm(x_sorted, w, ws: MoeWorkspace, rows: int):
    """`x_sorted [rows, K]` (rows sorted by expert), `w [E_local, N, K]` -> `[rows, N]`."""
    E, N, K = w.shape
    out = torch.empty((rows, N), dtype=x_sorted.dtype, device=x_sorted.device)
    sc = native.gemm_scratch(x_sorted.device)
    rc = _lib().sglb_grouped_gemm_bf16(x_sorted.data_ptr(), w.data_ptr(), out.data_ptr(), ws.offsets.data_ptr(),
                                       ws.tile_group.data_ptr(), ws.tile_row0.data_ptr(),
                                       ws.counts.data_ptr() + 4, rows, N, K, E, sc.workspace.data_ptr(), sc.bytes,
                                       sc.counters.data_ptr(), native._stream())
    native._check(rc, "grouped_gemm")
    return out


def grouped_gemm_fp8(xq_sorted, scale_x, wq, scale_w, ws: MoeWorkspace, rows: int):
    """e4m3 grouped GEMM on the tcgen05 `kind::f8f6f4` path: `xq_sorted [rows, K]` with per-row scales
    `scale_x [rows]`, `wq [E_local, N, K]` with per-output-channel scales `scale_w [E_local, N]` -> bf16 `[rows, N]`."""
    E, N, K = wq.shape
    assert xq_sorted.dtype == torch.float8_e4m3fn and wq.dtype == torch.float8_e4m3fn
    assert scale_x.dtype == torch.float32 and scale_w.dtype == torch.float32
    assert scale_x.numel() >= rows and scale_w.numel() == E * N and K % 16 == 0
    out = torch.empty((rows, N), dtype=torch.bfloat16, device=xq_sorted.device)
    sc = native.gemm_scratch(xq_sorted.device)
    rc = _lib().sglb_grouped_gemm_fp8(xq_sorted.data_ptr(), wq.data_ptr(), scale_x.data_ptr(), scale_w.data_ptr(),
                                      out.data_ptr(), ws.offsets.data_ptr(), ws.tile_group.data_ptr(),
                                      ws.tile_row0.data_ptr(), ws.counts.data_ptr() + 4, rows, N, K, E,
                                      sc.workspace.data_ptr(), sc.bytes, sc.counters.data_ptr(), native._stream())
    native._check(rc, "grouped_gemm_fp8")
    return out


def fused_experts_fp8(x, w13_q, w13_scale, w2_q, w2_scale, topk_weights, topk_ids, expert_start: int = 0,
                      ws: MoeWorkspace | None = None, add=None, out=None):
    """W8A8 e4m3 routed-expert FFN: align -> gather -> per-token quantise -> grouped fp8 GEMM (gate|up) ->
    fused SiLU*mul + per-token quantise -> grouped fp8 GEMM (down) -> weighted combine.  Weights are per-channel
    quantised (`w13_q [E_local, 2I, H]`, `w13_scale [E_local, 2I]`, `w2_q [E_local, H, I]`, `w2_scale [E_local, H]`)."""
    T, H = x.shape
    k = topk_ids.shape[1]
    E_local = w13_q.shape[0]
    pairs = T * k
    if ws is None or ws.max_pairs < pairs:
        ws = MoeWorkspace(pairs, E_local, x.device)
    moe_align(topk_ids, expert_start, E_local, ws)
    xs = moe_gather(x, ws, pairs)
    valid = ws.counts[0:1]
    xq, sx = native.quant_fp8_rows(xs, valid_rows=valid)
    h = grouped_gemm_fp8(xq, sx, w13_q, w13_scale, ws, pairs)
    aq, sa = native.quant_fp8_rows(h, gated=True, valid_rows=valid)
    y = grouped_gemm_fp8(aq, sa, w2_q, w2_scale, ws, pairs)
    return moe_combine(y, topk_weights, ws, T, add=add, out=out)


def grouped_gemm_fp8_block(xq_sorted, sx, wq, sw, ws: MoeWorkspace, rows: int):
    """Block-scaled e4m3 grouped GEMM: `xq_sorted [rows, K]` with group scales `sx [K/128, >=rows]`, `wq [E, N, K]`
    with `sw [E, N/128, K/128]` -> bf16 `[rows, N]` (`csrc/gemm_fp8_block.cu`)."""
    E, N, K = wq.shape
    out = torch.empty((rows, N), dtype=torch.bfloat16, device=xq_sorted.device)
    L = _lib()
    L.sglb_grouped_gemm_fp8_block.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    rc = L.sglb_grouped_gemm_fp8_block(xq_sorted.data_ptr(), wq.data_ptr(), sx.data_ptr(), sx.shape[1], sw.data_ptr(),
                                       out.data_ptr(), ws.offsets.data_ptr(), ws.tile_group.data_ptr(),
                                       ws.tile_row0.data_ptr(), ws.counts.data_ptr() + 4, rows, N, K, E,
                                       native._stream())
    native._check(rc, "grouped_gemm_fp8_block")
    return out


def fused_experts_fp8_block(x, w13_q, w13_scale, w2_q, w2_scale, topk_weights, topk_ids, expert_start: int = 0,
                            ws: MoeWorkspace | None = None, add=None, out=None):
    """Routed-expert FFN on 128 x 128 block-scaled e4m3 weights (DeepSeek-V3 format) with per-token-group-128
    activation scales: align -> gather -> group quantise -> grouped block GEMM (gate|up) -> SiLU*mul -> group
    quantise -> grouped block GEMM (down) -> weighted combine."""
    T, H = x.shape
    k = topk_ids.shape[1]
    E_local = w13_q.shape[0]
    pairs = T * k
    if ws is None or ws.max_pairs < pairs:
        ws = MoeWorkspace(pairs, E_local, x.device)
    moe_align(topk_ids, expert_start, E_local, ws)
    xs = moe_gather(x, ws, pairs)
    valid = ws.counts[0:1]
    xq, sx = native.quant_fp8_group128(xs, valid_rows=valid)
    h = grouped_gemm_fp8_block(xq, sx, w13_q, w13_scale, ws, pairs)
    a = native.silu_and_mul(h)
    aq, sa = native.quant_fp8_group128(a, valid_rows=valid)
    y = grouped_gemm_fp8_block(aq, sa, w2_q, w2_scale, ws, pairs)
    return moe_combine(y, topk_weights, ws, T, add=add, out=out)


def moe_combine(y_sorted, topk_weights, ws: MoeWorkspace, T: int, add=None, out=None):
    k = topk_weights.shape[1]
    H = y_sorted.shape[1]
    if out is None:
        out = torch.empty((T, H), dtype=y_sorted.dtype, device=y_sorted.device)
    rc = _lib().sglb_moe_combine(out.data_ptr(), y_sorted.data_ptr(), topk_weights.data_ptr(), ws.pair_row.data_ptr(),
                                 T, k, H, add.data_ptr() if add is not None else None, native._stream())
    native._check(rc, "moe_combine")
    return out


def fused_experts(x, w13, w2, topk_weights, topk_ids, expert_start: int = 0, ws: MoeWorkspace | None = None,
                  add=None, out=None):
    """Routed-expert FFN with the native kernels: align -> gather -> grouped GEMM (gate|up) -> SiLU*mul ->
    grouped GEMM (down) -> weighted combine.  `w13 [E_local, 2I, H]`, `w2 [E_local, H, I]`."""
    T, H = x.shape
    k = topk_ids.shape[1]
    E_local = w13.shape[0]
    pairs = T * k
    if ws is None or ws.max_pairs < pairs:
        ws = MoeWorkspace(pairs, E_local, x.device)
    moe_align(topk_ids, expert_start, E_local, ws)
    xs = moe_gather(x, ws, pairs)
    h = grouped_gemm(xs, w13, ws, pairs)
    a = native.silu_and_mul(h)
    y = grouped_gemm(a, w2, ws, pairs)
    return moe_combine(y, topk_weights, ws, T, add=add, out=out)
