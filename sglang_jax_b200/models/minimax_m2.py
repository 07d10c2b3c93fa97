"""MiniMax-M2 (reference `python/sgl_jax/srt/models/minimax_m2.py`): GQA attention whose q/k
RMSNorm spans the whole projection (all heads jointly) before RoPE, every layer a sigmoid-routed
MoE with a selection-only correction bias and renormalised top-k weights."""

from __future__ import annotations

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead, get_rope
from ..layers.fused_block import partial_add_norm, row_linear_add_norm
from ..layers.gate import GateLogit, TopK
from ..layers.layernorm import RMSNorm
from ..layers.linear import QKVParallelLinear, RowParallelLinear
from ..layers.logits_processor import LogitsProcessor
from ..layers.moe import FusedMoE
from ..layers.radix_attention import RadixAttention
from ..parallel import state as ps
from .llama import DenseModel, LlamaForCausalLM
from .moe_loading import load_sparse_weights


class _FullWidthNorm(nn.Module):
    """RMSNorm over a dimension that is split across tensor ranks: the mean of squares is
    reduced over the ranks, the weight is this rank's slice."""

    def __init__(self, full_dim: int, local_dim: int, eps: float, dtype, shard_rank: int):
        super().__init__()
        self.full_dim, self.local_dim, self.eps, self.shard_rank = full_dim, local_dim, eps, shard_rank
        self.weight = nn.Parameter(torch.ones(local_dim, dtype=dtype), requires_grad=False)

    def weight_loader(self, param, w, shard_id=None):
        param.data.copy_(w.narrow(0, self.shard_rank * self.local_dim, self.local_dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        ss = xf.pow(2).sum(-1, keepdim=True)
        if self.local_dim != self.full_dim:
            ss = ps.all_reduce(ss)
        return (xf * torch.rsqrt(ss / self.full_dim + self.eps)).to(x.dtype) * self.weight


class MiniMaxM2Attention(nn.Module):
    def __init__(self, config, layer_id, dtype):
        super().__init__()
        H = config.hidden_size
        self.head_dim = getattr(config, "head_dim", None) or H // config.num_attention_heads
        nh, nkv = config.num_attention_heads, config.num_key_value_heads
        self.qkv_proj = QKVParallelLinear(H, self.head_dim, nh, nkv, False, dtype)
        self.o_proj = RowParallelLinear(nh * self.head_dim, H, False, dtype)
        qp = self.qkv_proj
        eps = config.rms_norm_eps
        self.q_norm = _FullWidthNorm(nh * self.head_dim, qp.q_size, eps, dtype, qp.tp_rank)
        kv_rank = qp.tp_rank // qp.num_kv_head_replicas
        # replicated KV heads see the same slice on several ranks: reduce over distinct slices only
        self.k_norm = _FullWidthNorm(nkv * self.head_dim, qp.k_size, eps, dtype, kv_rank)
        self.kv_replicas = qp.num_kv_head_replicas
        rotary_dim = getattr(config, "rotary_dim", None) or int(self.head_dim * getattr(config, "partial_rotary_factor", 1.0))
        rp = getattr(config, "rope_parameters", None) or {}
        theta = getattr(config, "rope_theta", None) or rp.get("rope_theta", 10000.0)
        self.rotary_emb = get_rope(self.head_dim, rotary_dim, config.max_position_embeddings, theta, True, None, dtype)
        self.attn = RadixAttention(qp.num_heads, self.head_dim, self.head_dim ** -0.5, qp.num_kv_heads, layer_id)

    def forward(self, x, forward_batch):
        qp = self.qkv_proj
        qkv = qp(x)
        q, k, v = qkv.split([qp.q_size, qp.k_size, qp.v_size], dim=-1)
        k_n = self.k_norm(k) if self.kv_replicas == 1 else self._k_norm_replicated(k)
        qkv = torch.cat([self.q_norm(q), k_n, v], dim=-1)
        return self.attn(qkv, forward_batch, self.rotary_emb)

    def _k_norm_replicated(self, k):
        kf = k.float()
        ss = ps.all_reduce(kf.pow(2).sum(-1, keepdim=True)) / self.kv_replicas
        n = self.k_norm
        return (kf * torch.rsqrt(ss / n.full_dim + n.eps)).to(k.dtype) * n.weight


class MiniMaxM2MoE(nn.Module):
    def __init__(self, config, layer_id, dtype):
        super().__init__()
        E = config.num_local_experts
        self.gate = GateLogit(config.hidden_size, E, dtype, correction_bias=True, score_func="sigmoid")
        self.topk = TopK(config.num_experts_per_tok, renormalize=True, scoring_func="sigmoid")
        self.experts = FusedMoE(E, config.hidden_size, config.intermediate_size, dtype, layer_id=layer_id)
        self.tp_size = self.experts.tp_size

    def partial(self, x, out=None):
        w, ids = self.topk(self.gate(x), self.gate.e_score_correction_bias)
        return self.experts(x, w, ids, out=out)


class MiniMaxM2DecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype, **kw):
        super().__init__()
        eps = config.rms_norm_eps
        self.self_attn = MiniMaxM2Attention(config, layer_id, dtype)
        self.mlp = MiniMaxM2MoE(config, layer_id, dtype)
        self.input_layernorm = RMSNorm(config.hidden_size, eps, dtype)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps, dtype)

    def forward(self, h_normed, residual, fb, next_norm):
        a = self.self_attn(h_normed, fb)
        h, residual = row_linear_add_norm(self.self_attn.o_proj, a, residual, self.post_attention_layernorm)
        return partial_add_norm(lambda out: self.mlp.partial(h, out), h.shape[0], h.shape[1], residual, next_norm,
                                self.mlp.tp_size, block=self.mlp, x=h)


class MiniMaxM2Model(DenseModel):
    layer_cls = MiniMaxM2DecoderLayer


class MiniMaxM2ForCausalLM(LlamaForCausalLM):
    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        self.config = config
        self.dtype = dtype
        self.model = MiniMaxM2Model(config, dtype)
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        self.logits_processor = LogitsProcessor(config.vocab_size)
        self.capture_aux_hidden_states = False

    def load_weights(self, weights):
        return load_sparse_weights(
            self, weights,
            renames=[(".block_sparse_moe.", ".mlp."), (".mlp.e_score_correction_bias", ".mlp.gate.e_score_correction_bias")],
            expert_proj={"w1": "gate", "w3": "up", "w2": "down", "gate_proj": "gate", "up_proj": "up",
                         "down_proj": "down"})


EntryClass = [MiniMaxM2ForCausalLM]
