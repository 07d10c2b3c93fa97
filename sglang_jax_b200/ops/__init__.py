"""Hot ops of the model forward.

Every op has two implementations: the hand-written sm_100a kernel (module
`native`, a C-ABI shared library loaded with ctypes) and a plain-PyTorch statement
(module `reference`).  bf16 CUDA tensors take the native path; CPU tensors and other
dtypes take the reference path.  On a machine with a GPU the native library is
mandatory: if it cannot be loaded the first bf16 CUDA call raises instead of
quietly running the reference.
"""

from __future__ import annotations

import torch

from . import reference

_FORCE_REFERENCE = False


def set_force_reference(flag: bool):
    """Route every op through the PyTorch statements (debugging / `--disable-custom-kernels`)."""
    global _FORCE_REFERENCE
    _FORCE_REFERENCE = bool(flag)


def use_native(x: torch.Tensor) -> bool:
    return (not _FORCE_REFERENCE) and x.is_cuda and x.dtype == torch.bfloat16


def varlen_attention(q, k, v, seq_lens, scale: float):
    """Bidirectional attention over packed sequences (encoders, diffusion transformers)."""
    if use_native(q) and q.shape[-1] <= 128 and q.shape[1] % k.shape[1] == 0 and q.shape[1] // k.shape[1] <= 16 \
            and k.dtype == q.dtype and v.dtype == q.dtype:
        return _native().varlen_attention(q, k, v, seq_lens, scale)
    return reference.varlen_attention(q, k, v, seq_lens, scale)


def use_native_sampling(logits: torch.Tensor) -> bool:
    return (not _FORCE_REFERENCE) and logits.is_cuda and logits.dim() == 2 \
        and logits.dtype in (torch.float32, torch.bfloat16)


def _native():
    from . import native
    return native


def rmsnorm(x, w, eps, gemma=False):
    if use_native(x) and w.dtype == x.dtype:
        return _native().rmsnorm(x, w, eps, gemma)
    return reference.rmsnorm(x, w, eps, gemma)


def fused_add_rmsnorm(x, residual, w, eps, gemma=False):
    if use_native(x) and w.dtype == x.dtype:
        return _native().fused_add_rmsnorm(x, residual, w, eps, gemma)
    return reference.fused_add_rmsnorm(x, residual, w, eps, gemma)


def silu_and_mul(x):
    if use_native(x):
        return _native().silu_and_mul(x)
    return reference.silu_and_mul(x)


def linear(x, w, bias=None):
    if w.dtype != x.dtype and w.is_floating_point() and w.dtype.itemsize >= 2:
        # a per-module dtype (`--dtype-config`): compute in the weight's dtype, hand back the activations' dtype
        return reference.linear(x.to(w.dtype), w, bias.to(w.dtype) if bias is not None else None).to(x.dtype)
    if use_native(x) and w.dtype == torch.bfloat16:
        from ..parallel import state as ps
        comm = ps.get_state().fused_comm
        if comm is not None and comm.pending_gather is not None:
            # `x` may be a fused all-gather nobody has waited for yet: the GEMM waits per chunk of rows
            return comm.consume_linear(x, w, bias)
        return _native().linear(x, w, bias)
    return reference.linear(x, w, bias)


def rope_qknorm_kvwrite(qkv, positions, cos_sin, q_norm_w, k_norm_w, eps, num_q_heads, num_kv_heads,
                        head_dim, kv_buffer, out_cache_loc, page_size, is_neox=True, rotary_dim=None,
                        gemma_norm=False):
    if use_native(qkv) and (kv_buffer is None or kv_buffer.dtype == torch.bfloat16) and not gemma_norm:
        return _native().rope_qknorm_kvwrite(qkv, positions, cos_sin, q_norm_w, k_norm_w, eps, num_q_heads,
                                             num_kv_heads, head_dim, kv_buffer, out_cache_loc, page_size,
                                             is_neox, rotary_dim)
    return reference.rope_qknorm_kvwrite(qkv, positions, cos_sin, q_norm_w, k_norm_w, eps, num_q_heads,
                                         num_kv_heads, head_dim, kv_buffer, out_cache_loc, page_size,
                                         is_neox, rotary_dim, gemma_norm)


def paged_attention(q, kv_buffer, page_table, req_pool_indices, seq_lens, page_size, scale,
                    cu_q_lens=None, prefix_lens=None, sliding_window=0, soft_cap=0.0, sinks=None,
                    custom_mask=None, max_q_len=0, max_seq_len=0):
    compact_mask = custom_mask is None or (custom_mask.dim() == 3 and cu_q_lens is not None)
    if use_native(q) and kv_buffer.dtype == torch.bfloat16 and sinks is None and compact_mask \
            and q.shape[-1] in (64, 128):
        return _native().paged_attention(q, kv_buffer, page_table, req_pool_indices, seq_lens, page_size,
                                         scale, cu_q_lens, prefix_lens, sliding_window, soft_cap,
                                         max_q_len, max_seq_len, tail_mask=custom_mask)
    return reference.paged_attention(q, kv_buffer, page_table, req_pool_indices, seq_lens, page_size, scale,
                                     cu_q_lens, prefix_lens, sliding_window, soft_cap, sinks, custom_mask)


def embedding(ids, table, vocab_start=0, masked=False):
    if use_native(table) and ids.dtype == torch.int32:
        return _native().embedding(ids, table, vocab_start, masked)
    return reference.embedding(ids, table, vocab_start, masked)


def argmax(logits):
    """Greedy pick per row; the first maximal index wins."""
    if (not _FORCE_REFERENCE) and logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16):
        return _native().argmax(logits)
    return torch.argmax(logits, dim=-1).to(torch.int32)


def topk_route(router_logits, top_k, scoring="softmax", renormalize=True, correction_bias=None,
               num_expert_group=0, topk_group=0, routed_scaling_factor=1.0):
    if (not _FORCE_REFERENCE) and router_logits.is_cuda and router_logits.shape[-1] <= 512 and top_k <= 16 \
            and router_logits.dtype in (torch.float32, torch.bfloat16):
        from . import moe_native
        return moe_native.topk_route(router_logits, top_k, scoring, renormalize, correction_bias,
                                     num_expert_group, topk_group, routed_scaling_factor)
    return reference.topk_route(router_logits, top_k, scoring, renormalize, correction_bias,
                                num_expert_group, topk_group, routed_scaling_factor)


def fused_experts(x, w13, w2, topk_weights, topk_ids, expert_start=0, workspace=None, add=None):
    """Routed-expert FFN: `w13 [E_local, 2I, H]` (gate rows then up rows), `w2 [E_local, H, I]`."""
    if use_native(x) and w13.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and w2.shape[-1] % 8 == 0:
        from . import moe_native
        return moe_native.fused_experts(x, w13, w2, topk_weights, topk_ids, expert_start, workspace, add)
    y = reference.moe_forward(x, w13, w2, topk_weights, topk_ids, expert_start)
    return y if add is None else (y.float() + add.float()).to(y.dtype)


def mla_paged_attention(q_latent, q_pe, kv_buffer, page_table, req_pool_indices, seq_lens, page_size, scale,
                        kv_lora_rank, cu_q_lens=None, prefix_lens=None, allowed=None, max_seq_len=0):
    """Absorbed-MLA attention over the latent cache `[pages, P, kv_lora_rank + rope_dim]`."""
    if use_native(q_latent) and cu_q_lens is None and allowed is None and req_pool_indices.dtype == torch.int32 \
            and _native().mla_decode_supported(q_latent, q_pe, kv_buffer, kv_lora_rank, page_size):
        return _native().mla_decode(q_latent, q_pe, kv_buffer, page_table, req_pool_indices, seq_lens, page_size,
                                    scale, max_seq_len)
    return reference.mla_paged_attention(q_latent, q_pe, kv_buffer, page_table, req_pool_indices, seq_lens,
                                         page_size, scale, kv_lora_rank, cu_q_lens, prefix_lens, allowed)
