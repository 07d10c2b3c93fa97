"""Plain-PyTorch statements of every hot op.

These are (1) the CPU execution path, (2) the fp32 oracles the CUDA kernels are
tested against, and (3) the semantics documentation of each op.  Attention
semantics follow the reference's `NativeAttention.forward_attention`
(`python/sgl_jax/srt/layers/attention/native_backend.py:169-435`): causal over
``prefix_len + i`` in extend mode, decode attends to ``seq_len`` keys, GQA by
repeating KV heads, optional sliding window / logit soft-cap / sink term.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, gemma: bool = False) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    wf = w.float() + 1.0 if gemma else w.float()
    return (y * wf).to(x.dtype)


def fused_add_rmsnorm(x, residual, w, eps, gemma: bool = False):
    """residual' = x + residual (rounded to the activation dtype); y = rmsnorm(residual')."""
    r = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(r, w, eps, gemma), r


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    return (F.silu(x[..., :d].float()) * x[..., d:].float()).to(x.dtype)


def gelu_and_mul(x: torch.Tensor, approximate: str = "tanh") -> torch.Tensor:
    d = x.shape[-1] // 2
    return (F.gelu(x[..., :d].float(), approximate=approximate) * x[..., d:].float()).to(x.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ w.T (+ bias); `w` is `[out, in]` as stored in HF checkpoints."""
    return F.linear(x, w, bias)


def build_cos_sin_cache(rotary_dim: int, max_pos: int, base: float, inv_freq: torch.Tensor | None = None,
                        mscale: float = 1.0, device=None) -> torch.Tensor:
    """fp32 `[max_pos, rotary_dim]`: first half cos, second half sin.  Computed on the host in
    fp32 and then moved to `device` (default: the ambient default device)."""
    if device is None:
        device = torch.empty(0).device
    if inv_freq is None:
        inv_freq = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32, device="cpu") / rotary_dim))
    t = torch.arange(max_pos, dtype=torch.float32, device="cpu")
    freqs = torch.outer(t, inv_freq.float().cpu())
    return torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1).to(device)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor, is_neox: bool = True,
               rotary_dim: int | None = None) -> torch.Tensor:
    """x `[T, H, D]`; rotates the first `rotary_dim` lanes of every head."""
    D = x.shape[-1]
    rd = rotary_dim or D
    cs = cos_sin[positions.long()]
    cos, sin = cs[:, : rd // 2].unsqueeze(1), cs[:, rd // 2:].unsqueeze(1)
    xr = x[..., :rd].float()
    if is_neox:
        x1, x2 = xr[..., : rd // 2], xr[..., rd // 2:]
        out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
    else:
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).flatten(-2)
    if rd < D:
        out = torch.cat([out, x[..., rd:].float()], dim=-1)
    return out.to(x.dtype)


def rope_qknorm_kvwrite(qkv, positions, cos_sin, q_norm_w, k_norm_w, eps, num_q_heads, num_kv_heads,
                        head_dim, kv_buffer, out_cache_loc, page_size, is_neox=True, rotary_dim=None,
                        gemma_norm: bool = False):
    """Split fused qkv, per-head RMSNorm on q and k (Qwen3), RoPE, write K/V rows into the
    paged cache `[pages, 2, Hkv, P, D]`; returns roped q `[T, Hq, D]`."""
    T = qkv.shape[0]
    qs, ks = num_q_heads * head_dim, num_kv_heads * head_dim
    q = qkv[:, :qs].reshape(T, num_q_heads, head_dim)
    k = qkv[:, qs:qs + ks].reshape(T, num_kv_heads, head_dim)
    v = qkv[:, qs + ks:].reshape(T, num_kv_heads, head_dim)
    if q_norm_w is not None:
        q = rmsnorm(q, q_norm_w, eps, gemma_norm)
    if k_norm_w is not None:
        k = rmsnorm(k, k_norm_w, eps, gemma_norm)
    if cos_sin is not None:
        q = apply_rope(q, positions, cos_sin, is_neox, rotary_dim)
        k = apply_rope(k, positions, cos_sin, is_neox, rotary_dim)
    if kv_buffer is not None:
        page = (out_cache_loc // page_size).long()
        off = (out_cache_loc % page_size).long()
        kv_buffer[page, 0, :, off] = k.to(kv_buffer.dtype)
        kv_buffer[page, 1, :, off] = v.to(kv_buffer.dtype)
    return q.contiguous()


def gather_kv(kv_buffer, page_table, req_idx: int, seq_len: int, page_size: int):
    """K,V `[seq_len, Hkv, D]` of one request from the paged cache."""
    n_pages = (seq_len + page_size - 1) // page_size
    pages = page_table[req_idx, :n_pages].long()
    blk = kv_buffer[pages]                       # [n, 2, H, P, D]
    k = blk[:, 0].permute(0, 2, 1, 3).reshape(-1, blk.shape[2], blk.shape[4])[:seq_len]
    v = blk[:, 1].permute(0, 2, 1, 3).reshape(-1, blk.shape[2], blk.shape[4])[:seq_len]
    return k, v


def paged_attention(q, kv_buffer, page_table, req_pool_indices, seq_lens, page_size, scale,
                    cu_q_lens=None, prefix_lens=None, sliding_window: int = 0, soft_cap: float = 0.0,
                    sinks: torch.Tensor | None = None, custom_mask: torch.Tensor | None = None,
                    compute_dtype=torch.float32):
    """Ragged causal GQA attention over the paged cache (which already holds this step's K/V).

    decode: `cu_q_lens is None`, one query row per sequence.
    extend: rows `cu_q_lens[b]:cu_q_lens[b+1]` belong to sequence b and sit at positions
    `prefix_lens[b] + i`."""
    T, Hq, D = q.shape
    out = torch.empty_like(q)
    B = len(req_pool_indices)
    rp = req_pool_indices.tolist()
    sl = seq_lens.tolist()
    cu = cu_q_lens.tolist() if cu_q_lens is not None else list(range(B + 1))
    pre = prefix_lens.tolist() if prefix_lens is not None else [s - 1 for s in sl]
    mask_off = 0
    for b in range(B):
        q0, q1 = cu[b], cu[b + 1]
        n = q1 - q0
        if n == 0:
            continue
        S = sl[b]
        k, v = gather_kv(kv_buffer, page_table, rp[b], S, page_size)
        Hkv = k.shape[1]
        g = Hq // Hkv
        qb = q[q0:q1].to(compute_dtype).view(n, Hkv, g, D)
        kf, vf = k.to(compute_dtype), v.to(compute_dtype)
        logits = torch.einsum("nhgd,shd->hgns", qb, kf) * scale
        if soft_cap and soft_cap > 0:
            logits = soft_cap * torch.tanh(logits / soft_cap)
        qpos = torch.arange(pre[b], pre[b] + n, device=q.device).view(n, 1)
        kpos = torch.arange(S, device=q.device).view(1, S)
        allowed = kpos <= qpos
        if sliding_window and sliding_window > 0:
            allowed &= kpos > qpos - sliding_window
        if custom_mask is not None and custom_mask.dim() == 3:
            # compact form [B, q, tail]: the last `tail` keys follow the mask, earlier keys are visible
            tail = custom_mask.shape[2]
            allowed = torch.ones(n, S, dtype=torch.bool, device=q.device)
            allowed[:, S - tail:] = custom_mask[b, :n].bool()
        elif custom_mask is not None:
            m = custom_mask[mask_off:mask_off + n * S].view(n, S).bool()
            mask_off += n * S
            allowed = m
        logits = logits.masked_fill(~allowed.view(1, 1, n, S), float("-inf"))
        if sinks is not None:
            sink = sinks.to(compute_dtype).view(Hkv, g, 1, 1).expand(Hkv, g, n, 1)
            full = torch.cat([logits, sink], dim=-1)
            p = torch.softmax(full.float(), dim=-1)[..., :-1].to(compute_dtype)
        else:
            p = torch.softmax(logits.float(), dim=-1).to(compute_dtype)
        o = torch.einsum("hgns,shd->nhgd", p, vf)
        out[q0:q1] = o.reshape(n, Hq, D).to(q.dtype)
    return out


# ----------------------------------------------------------------------------- sampling
def apply_token_bitmask(logits: torch.Tensor, bitmask: torch.Tensor) -> torch.Tensor:
    """bitmask int32 `[B, ceil(V/32)]`, bit set = token allowed."""
    V = logits.shape[-1]
    bits = (bitmask.unsqueeze(-1) >> torch.arange(32, device=bitmask.device, dtype=torch.int32)) & 1
    allowed = bits.reshape(bitmask.shape[0], -1)[:, :V].bool()
    return logits.masked_fill(~allowed, float("-inf"))


def _i32(x: torch.Tensor) -> torch.Tensor:
    """Wrap int64 arithmetic to signed 32-bit."""
    return ((x + 2 ** 31) % 2 ** 32) - 2 ** 31


def multinomial_with_seed(probs: torch.Tensor, seeds: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Batch-invariant seeded sampling by hashed Gumbel-max, reproducing the reference's
    int32-wraparound hash (`python/sgl_jax/srt/layers/sampler.py:250-293`):
    step_seed = seed*19349663 ^ position*73856093; hash = step_seed*805306457 ^ col*479001599;
    u = (hash mod 2^24)/2^24; argmax(log(p+1e-9) + gumbel(u))."""
    B, V = probs.shape
    s = seeds.to(torch.int64).view(B, 1)
    pos = positions.to(torch.int64).view(B, 1)
    step_seed = _i32(_i32(s * 19349663) ^ _i32(pos * 73856093))
    col = torch.arange(V, device=probs.device, dtype=torch.int64).view(1, V)
    h = _i32(_i32(step_seed * 805306457) ^ _i32(col * 479001599))
    u = (h % (1 << 24)).float() / float(1 << 24)
    eps = 1e-9
    gumbel = -torch.log(-torch.log(u + eps) + eps)
    return torch.argmax(torch.log(probs.float() + eps) + gumbel, dim=-1)


def top_k_top_p_min_p_probs(logits, temperatures, top_ks, top_ps, min_ps):
    """fp32 probabilities after temperature, top-k, top-p and min-p filtering (renormalised)."""
    lf = logits.float() / temperatures.view(-1, 1).clamp_min(1e-6)
    probs = torch.softmax(lf, dim=-1)
    sp, si = probs.sort(dim=-1, descending=True)
    V = probs.shape[-1]
    ranks = torch.arange(V, device=probs.device).view(1, -1)
    keep = ranks < top_ks.view(-1, 1).clamp(max=V)
    cum = sp.cumsum(-1)
    keep &= (cum - sp) < top_ps.view(-1, 1)
    keep &= sp >= sp[:, :1] * min_ps.view(-1, 1)
    keep[:, 0] = True
    sp = sp * keep
    sp = sp / sp.sum(-1, keepdim=True)
    out = torch.zeros_like(probs)
    out.scatter_(1, si, sp)
    return out


def varlen_attention(q, k, v, seq_lens, scale: float):
    """Bidirectional attention inside each sequence of a packed ragged batch: `q [T, Hq, D]`, `k, v [T, Hkv, D]`,
    `seq_lens` host ints.  fp32 softmax."""
    out = torch.empty_like(q)
    g = q.shape[1] // k.shape[1]
    o = 0
    for n in (int(x) for x in seq_lens):
        if n == 0:
            continue
        qq = q[o:o + n].float().transpose(0, 1)                                  # [Hq, n, D]
        kk = k[o:o + n].float().transpose(0, 1).repeat_interleave(g, 0)
        vv = v[o:o + n].float().transpose(0, 1).repeat_interleave(g, 0)
        p = torch.softmax(qq @ kk.transpose(1, 2) * scale, dim=-1)
        out[o:o + n] = (p @ vv).transpose(0, 1).to(q.dtype)
        o += n
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0, masked: bool = False) -> torch.Tensor:
    """Row lookup.  With `masked` (vocab-parallel shard) ids outside
    `[vocab_start, vocab_start + rows)` produce zero rows so an all-reduce completes them."""
    if not masked:
        return table[ids.long()]
    local = ids.long() - vocab_start
    ok = (local >= 0) & (local < table.shape[0])
    out = table[local.clamp(0, table.shape[0] - 1)]
    return out * ok.unsqueeze(-1).to(out.dtype)


# ----------------------------------------------------------------------------- MoE
def topk_route(router_logits, top_k, scoring="softmax", renormalize=True, correction_bias=None,
               num_expert_group=0, topk_group=0, routed_scaling_factor=1.0):
    """Router semantics of the reference (`python/sgl_jax/srt/layers/gate.py:59-333`):
    scores = softmax/sigmoid of fp32 logits; biased: choose by score+bias, weight = unbiased
    score; grouped: group score = max (unbiased) or sum of top-2 (biased), keep `topk_group`
    groups, then top-k; optional renormalise; times `routed_scaling_factor`."""
    lf = router_logits.float()
    if scoring == "softmax":
        scores = torch.softmax(lf, dim=-1)
    elif scoring == "sigmoid":
        scores = torch.sigmoid(lf)
    elif scoring == "tanh":
        scores = torch.tanh(lf)
    else:
        raise ValueError(scoring)
    choose = scores + correction_bias.float() if correction_bias is not None else scores
    T, E = scores.shape
    if num_expert_group and num_expert_group > 1:
        gs = choose.view(T, num_expert_group, E // num_expert_group)
        if correction_bias is not None:
            group_scores = gs.topk(2, dim=-1).values.sum(-1)
        else:
            group_scores = gs.max(-1).values
        gidx = group_scores.topk(topk_group, dim=-1).indices
        gmask = torch.zeros_like(group_scores).scatter_(1, gidx, 1.0)
        mask = gmask.unsqueeze(-1).expand(T, num_expert_group, E // num_expert_group).reshape(T, E)
        choose = choose.masked_fill(mask == 0, float("-inf"))
    ids = choose.topk(top_k, dim=-1).indices
    w = scores.gather(1, ids)
    if renormalize:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    w = w * routed_scaling_factor
    return w, ids.to(torch.int32)


def moe_forward(x, w13, w2, topk_weights, topk_ids, expert_start: int = 0, act="silu"):
    """Dense statement of the routed-expert FFN.  `w13 [E_local, 2I, H]` (gate then up),
    `w2 [E_local, H, I]`; tokens routed to experts outside
    `[expert_start, expert_start + E_local)` contribute nothing (expert parallelism)."""
    T, H = x.shape
    out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    E_local = w13.shape[0]
    for e in range(E_local):
        sel = (topk_ids == e + expert_start)
        tok, slot = sel.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = F.linear(x[tok], w13[e])
        h = silu_and_mul(h) if act == "silu" else gelu_and_mul(h)
        y = F.linear(h, w2[e]).float()
        out.index_add_(0, tok, y * topk_weights[tok, slot].unsqueeze(-1).float())
    return out.to(x.dtype)


def grouped_gemm(x, w, group_sizes):
    """`x [M, K]` rows sorted by group, `w [E, N, K]`, `group_sizes [E]` -> `[M, N]`."""
    out = torch.empty((x.shape[0], w.shape[1]), dtype=x.dtype, device=x.device)
    o = 0
    for e, n in enumerate(group_sizes.tolist()):
        if n:
            out[o:o + n] = F.linear(x[o:o + n], w[e])
        o += n
    return out


# ----------------------------------------------------------------------------- MLA
def mla_paged_attention(q_nope_latent, q_pe, kv_buffer, page_table, req_pool_indices, seq_lens,
                        page_size, scale, kv_lora_rank, cu_q_lens=None, prefix_lens=None, allowed=None):
    """Absorbed MLA: every head attends over the shared latent cache
    `[pages, P, kv_lora_rank + rope_dim]`; logits = q_latent·c + q_pe·k_pe; output stays
    latent `[T, H, kv_lora_rank]` (caller applies W_UV).  `allowed[b]` (bool `[n_b, S_b]`) restricts
    request b's queries to the keys a sparse-attention indexer selected."""
    T, H, R = q_nope_latent.shape
    out = torch.empty_like(q_nope_latent)
    B = len(req_pool_indices)
    rp, sl = req_pool_indices.tolist(), seq_lens.tolist()
    cu = cu_q_lens.tolist() if cu_q_lens is not None else list(range(B + 1))
    pre = prefix_lens.tolist() if prefix_lens is not None else [s - 1 for s in sl]
    for b in range(B):
        q0, q1 = cu[b], cu[b + 1]
        n = q1 - q0
        if n == 0:
            continue
        S = sl[b]
        n_pages = (S + page_size - 1) // page_size
        rows = kv_buffer[page_table[rp[b], :n_pages].long()].reshape(-1, kv_buffer.shape[-1])[:S].float()
        c, kpe = rows[:, :kv_lora_rank], rows[:, kv_lora_rank:]
        logits = (torch.einsum("nhr,sr->hns", q_nope_latent[q0:q1].float(), c)
                  + torch.einsum("nhd,sd->hns", q_pe[q0:q1].float(), kpe)) * scale
        qpos = torch.arange(pre[b], pre[b] + n, device=logits.device).view(n, 1)
        kpos = torch.arange(S, device=logits.device).view(1, S)
        keep = kpos <= qpos
        if allowed is not None and allowed[b] is not None:      # sparse attention: [n, S] selected keys
            keep = keep & allowed[b]
        logits = logits.masked_fill(~keep.view(1, n, S), float("-inf"))
        p = torch.softmax(logits, dim=-1)
        out[q0:q1] = torch.einsum("hns,sr->nhr", p, c).to(out.dtype)
    return out
