"""GLM-5 (`GlmMoeDsaForCausalLM`): DeepSeek-style latent attention and sigmoid-routed experts, plus
a sparse-attention indexer per layer (reference `python/sgl_jax/srt/models/glm5_moe.py`:
`GlmDsaIndexer` :130, `Glm5Attention` :252).

The indexer owns light projections — `wq_b` from the query's low-rank residual to
`index_n_heads x index_head_dim`, a single-head key `wk` with a LayerNorm, and per-head weights
`weights_proj` — with NeoX RoPE on the first `qk_rope_head_dim` lanes.  Its key is cached per
token next to the latent row.  A query's score for key t is
`sum_h w_h * relu(q_h . k_t) * index_head_dim^-0.5 * index_n_heads^-0.5`; the `index_topk`
best causal keys are the only ones the main attention may see.  While a sequence is no longer
than `index_topk` the selection is every causal key, so the dense kernels run unchanged and
only the indexer keys are written.  (The checkpoint's Hadamard rotation of q and k is
orthogonal and leaves the scores unchanged; it is skipped.)
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from ..layers.embeddings import get_rope
from ..layers.linear import ReplicatedLinear
from ..ops import reference
from .deepseek_v3 import DeepseekV3ForCausalLM, MLAAttention


class _KeyNorm(nn.Module):
    """LayerNorm (scale and shift) over the indexer key."""

    def __init__(self, dim, dtype, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype), requires_grad=False)
        self.eps = eps

    def weight_loader(self, param, w, shard_id=None):
        param.data.copy_(w)

    def forward(self, x):
        return F.layer_norm(x.float(), x.shape[-1:], self.weight.float(), self.bias.float(), self.eps).to(x.dtype)


class GlmDsaIndexer(nn.Module):
    def __init__(self, config, dtype):
        super().__init__()
        self.n_heads, self.head_dim = config.index_n_heads, config.index_head_dim
        self.rope_dim = config.qk_rope_head_dim
        self.topk = int(config.index_topk)
        self.wq_b = ReplicatedLinear(config.q_lora_rank, self.n_heads * self.head_dim, False, dtype)
        self.wk = ReplicatedLinear(config.hidden_size, self.head_dim, False, dtype)
        self.k_norm = _KeyNorm(self.head_dim, dtype)
        self.weights_proj = ReplicatedLinear(config.hidden_size, self.n_heads, False, dtype)
        self.rotary_emb = get_rope(self.rope_dim, self.rope_dim, config.max_position_embeddings,
                                   getattr(config, "rope_theta", 10000.0), True, None, dtype)
        self.scale = self.head_dim ** -0.5 * self.n_heads ** -0.5

    def project(self, x, q_resid, positions):
        cs = self.rotary_emb.cos_sin_cache
        q = self.wq_b(q_resid).view(-1, self.n_heads, self.head_dim)
        k = self.k_norm(self.wk(x)).unsqueeze(1)
        r = self.rope_dim
        q = torch.cat([reference.apply_rope(q[..., :r], positions, cs, True), q[..., r:]], dim=-1)
        k = torch.cat([reference.apply_rope(k[..., :r], positions, cs, True), k[..., r:]], dim=-1).squeeze(1)
        return q, k, self.weights_proj(x).float() * self.scale

    def select(self, q, w, keys, first_pos: int):
        """`q [n, H, D]`, `w [n, H]`, `keys [S, D]` -> bool `[n, S]` of the selected causal keys."""
        n, S = q.shape[0], keys.shape[0]
        score = torch.einsum("nhs,nh->ns", torch.relu(torch.einsum("nhd,sd->nhs", q.float(), keys.float())), w)
        qpos = torch.arange(first_pos, first_pos + n, device=q.device).view(n, 1)
        score = score.masked_fill(torch.arange(S, device=q.device).view(1, S) > qpos, float("-inf"))
        idx = score.topk(min(self.topk, S), dim=-1).indices
        return torch.zeros(n, S, dtype=torch.bool, device=q.device).scatter_(1, idx, True)


class Glm5Attention(MLAAttention):
    def __init__(self, config, layer_id, dtype):
        super().__init__(config, layer_id, dtype)
        self.indexer = GlmDsaIndexer(config, dtype)
        self.select_keys = self._select_keys

    def _select_keys(self, x, q_resid, fb):
        ix = self.indexer
        q, k, w = ix.project(x, q_resid, fb.positions)
        pool = fb.token_to_kv_pool
        kbuf = pool.get_index_k_buffer(self.layer_id)
        kbuf[fb.out_cache_loc.long()] = k.to(kbuf.dtype)
        if fb.max_seq_len <= ix.topk:
            return None                       # every causal key is selected: plain dense attention
        B = len(fb.req_pool_indices)
        sl = fb.seq_lens.tolist()
        rp = fb.req_pool_indices.tolist()
        decode = fb.forward_mode.is_decode()
        cu = list(range(B + 1)) if decode else fb.cu_q_lens.tolist()
        pre = [s - 1 for s in sl] if decode else fb.extend_prefix_lens.tolist()
        P = fb.page_size
        out = []
        for b in range(B):
            S, q0, q1 = sl[b], cu[b], cu[b + 1]
            if S <= ix.topk or q1 == q0:
                out.append(None)
                continue
            pages = fb.page_table[rp[b], : (S + P - 1) // P].long()
            slots = (pages.view(-1, 1) * P + torch.arange(P, device=pages.device).view(1, P)).reshape(-1)[:S]
            out.append(ix.select(q[q0:q1], w[q0:q1], kbuf[slots], pre[b]))
        return out


def _patch(config):
    rp = getattr(config, "rope_parameters", None)
    if isinstance(rp, dict) and rp.get("rope_theta") and not getattr(config, "rope_theta", None):
        config.rope_theta = rp["rope_theta"]
    types = getattr(config, "mlp_layer_types", None)
    if types:
        config.first_k_dense_replace = next((i for i, t in enumerate(types) if t == "sparse"), len(types))
        config.moe_layer_freq = 1
    if not getattr(config, "topk_method", None):
        config.topk_method = "noaux_tc"
    if not getattr(config, "scoring_func", None):
        config.scoring_func = "sigmoid"
    return config


class GlmMoeDsaForCausalLM(DeepseekV3ForCausalLM):
    attn_cls = Glm5Attention

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__(_patch(config), dtype, quant_config)
        self.index_head_dim = int(config.index_head_dim)


class Glm5ForCausalLM(GlmMoeDsaForCausalLM):
    pass


EntryClass = [GlmMoeDsaForCausalLM, Glm5ForCausalLM]
