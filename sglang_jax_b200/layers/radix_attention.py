"""Attention layer over the paged KV cache.

The reference's `RadixAttention` (`python/sgl_jax/srt/layers/radix_attention.py:24`)
forwards to a pluggable backend (FlashAttention Pallas kernel / native jnp).  Here the
layer owns the whole per-token pipeline — q/k RMSNorm, RoPE, KV-cache write and ragged
paged attention — because on B200 the first three are one fused kernel and the KV write
must precede attention on the same stream anyway.  `attention_backend="native"` routes
the same calls through the PyTorch statements in `ops.reference`.
"""

from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..ops import reference


class RadixAttention(nn.Module):
    def __init__(self, num_heads: int, head_dim: int, scaling: float, num_kv_heads: int, layer_id: int,
                 sliding_window_size: int = 0, logit_cap: float = 0.0, v_head_dim: int | None = None):
        super().__init__()
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.v_head_dim = v_head_dim or head_dim
        self.scaling = scaling
        self.layer_id = layer_id
        self.sliding_window_size = sliding_window_size or 0
        self.logit_cap = logit_cap or 0.0

    def forward(self, qkv: torch.Tensor, forward_batch, rotary_emb=None, q_norm=None, k_norm=None,
                sinks: torch.Tensor | None = None, gemma_norm: bool = False) -> torch.Tensor:
        fb = forward_batch
        pool = fb.token_to_kv_pool
        kv_buffer = pool.get_kv_buffer(self.layer_id)
        loc = fb.out_cache_loc
        if hasattr(pool, "is_swa_layer") and pool.is_swa_layer(self.layer_id):
            loc = pool.translate_loc_from_full_to_swa(loc)
        native_backend = getattr(fb.attn_backend, "name", "fa") == "native"
        rope = ops.rope_qknorm_kvwrite if not native_backend else reference.rope_qknorm_kvwrite
        attn = ops.paged_attention if not native_backend else reference.paged_attention
        eps = q_norm.variance_epsilon if q_norm is not None else 1e-6
        mpos = fb.extras.get("mrope_positions") if hasattr(rotary_emb, "mrope_section") else None
        if mpos is not None:
            # multimodal rotary: the frequency lanes are driven by three position streams, so the
            # rotation is applied here and the fused kernel only normalises and writes the cache
            qs, ks = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
            q3 = qkv[:, :qs].reshape(-1, self.num_heads, self.head_dim)
            k3 = qkv[:, qs:qs + ks].reshape(-1, self.num_kv_heads, self.head_dim)
            if q_norm is not None:
                q3, k3 = q_norm(q3), k_norm(k3)
                q_norm = k_norm = None
            q3, k3 = rotary_emb(mpos, q3, k3)
            qkv = torch.cat([q3.flatten(1), k3.flatten(1), qkv[:, qs + ks:]], dim=-1)
            rotary_emb = None
        q = rope(qkv, fb.positions,
                 rotary_emb.cos_sin_cache if rotary_emb is not None else None,
                 q_norm.weight if q_norm is not None else None,
                 k_norm.weight if k_norm is not None else None,
                 eps, self.num_heads, self.num_kv_heads, self.head_dim, kv_buffer, loc, fb.page_size,
                 rotary_emb.is_neox_style if rotary_emb is not None else True,
                 rotary_emb.rotary_dim if rotary_emb is not None else None, gemma_norm)
        page_table = fb.page_table
        if hasattr(pool, "is_swa_layer") and pool.is_swa_layer(self.layer_id):
            page_table = fb.extras["swa_page_table"]
        kw = {}
        if not native_backend:
            kw = dict(max_q_len=fb.max_extend_len, max_seq_len=fb.max_seq_len)
        if fb.forward_mode.is_decode():
            out = attn(q, kv_buffer, page_table, fb.req_pool_indices, fb.seq_lens, fb.page_size, self.scaling,
                       None, None, self.sliding_window_size, self.logit_cap, sinks,
                       None, **kw)
        else:
            mask = fb.spec_info.custom_mask if (fb.spec_info is not None and
                                                getattr(fb.spec_info, "custom_mask", None) is not None) else None
            nd = int(getattr(fb, "num_decode_in_mixed", 0) or 0)
            B = fb.req_pool_indices.shape[0]
            if nd > 0 and mask is None and nd < B:
                # mixed step: the trailing `nd` requests are one-token decodes.  They go through the decode kernel
                # (split-KV over their whole context) instead of occupying a 128-row query tile each in the
                # prefill kernel; the leading requests are ordinary prefill rows.
                np_ = B - nd
                tp = q.shape[0] - nd
                out_p = attn(q[:tp], kv_buffer, page_table, fb.req_pool_indices[:np_], fb.seq_lens[:np_], fb.page_size,
                             self.scaling, fb.cu_q_lens[:np_ + 1], fb.extend_prefix_lens[:np_],
                             self.sliding_window_size, self.logit_cap, sinks, None, **kw)
                out_d = attn(q[tp:], kv_buffer, page_table, fb.req_pool_indices[np_:], fb.seq_lens[np_:], fb.page_size,
                             self.scaling, None, None, self.sliding_window_size, self.logit_cap, sinks, None, **kw)
                out = torch.cat([out_p.reshape(tp, -1), out_d.reshape(nd, -1)], dim=0)
            else:
                out = attn(q, kv_buffer, page_table, fb.req_pool_indices, fb.seq_lens, fb.page_size, self.scaling,
                           fb.cu_q_lens, fb.extend_prefix_lens, self.sliding_window_size, self.logit_cap, sinks,
                           mask, **kw)
        return out.reshape(out.shape[0], self.num_heads * self.head_dim)


class AttentionBackend:
    """Names the attention implementation a runner uses ("fa" = sm_100a kernels,
    "native" = PyTorch statements)."""

    def __init__(self, name: str):
        self.name = name
