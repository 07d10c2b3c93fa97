"""DeepSeek-V2 / V3 / R1: multi-head latent attention (absorbed form over a shared latent KV cache)
and group-limited sigmoid-routed experts with a shared expert.

Reference: `python/sgl_jax/srt/models/deepseek_v3.py` (absorbed MLA :302-370, MoE :497,
`patch_model_config` :723).  The cache holds one `kv_lora_rank + qk_rope_head_dim` row per token
(`mem_cache/memory_pool.py: MLATokenToKVPool`); queries are projected into the latent space with
W_UK, attention runs as multi-query attention over the latent rows, and W_UV maps the latent
output back to value heads.
"""

from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding, get_rope, yarn_get_mscale
from ..layers.fused_block import partial_add_norm, row_linear_add_norm
from ..layers.gate import GateLogit, TopK
from ..layers.layernorm import RMSNorm
from ..layers.linear import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear
from ..layers.logits_processor import LogitsProcessor
from ..layers.moe import FusedMoE
from ..ops import reference
from ..parallel import state as ps
from .llama import DenseMLP


class MLAAttention(nn.Module):
    def __init__(self, config, layer_id: int, dtype):
        super().__init__()
        self.layer_id = layer_id
        H = config.hidden_size
        self.tp = ps.tp_size()
        self.num_heads = config.num_attention_heads
        self.local_heads = self.num_heads // self.tp
        self.nope, self.rope_dim, self.v_dim = config.qk_nope_head_dim, config.qk_rope_head_dim, config.v_head_dim
        self.kv_lora = config.kv_lora_rank
        self.q_lora = getattr(config, "q_lora_rank", None)
        qk = self.nope + self.rope_dim
        eps = config.rms_norm_eps
        if self.q_lora:
            self.q_a_proj = ReplicatedLinear(H, self.q_lora, False, dtype)
            self.q_a_layernorm = RMSNorm(self.q_lora, eps, dtype)
            self.q_b_proj = ColumnParallelLinear(self.q_lora, self.num_heads * qk, False, dtype)
        else:
            self.q_proj = ColumnParallelLinear(H, self.num_heads * qk, False, dtype)
        self.kv_a_proj_with_mqa = ReplicatedLinear(H, self.kv_lora + self.rope_dim, False, dtype)
        self.kv_a_layernorm = RMSNorm(self.kv_lora, eps, dtype)
        self.kv_b_proj = ColumnParallelLinear(self.kv_lora, self.num_heads * (self.nope + self.v_dim), False, dtype)
        self.o_proj = RowParallelLinear(self.num_heads * self.v_dim, H, False, dtype)
        rs = getattr(config, "rope_scaling", None)
        if isinstance(rs, dict) and rs.get("rope_type", rs.get("type")) == "yarn":
            rs = dict(rs, rope_type="deepseek_yarn")
        # checkpoints store the rotary lanes interleaved; `rope_interleave=False` selects split-half
        self.rope_neox = not getattr(config, "rope_interleave", True)
        self.rotary_emb = get_rope(self.rope_dim, self.rope_dim, config.max_position_embeddings,
                                   getattr(config, "rope_theta", 10000.0), self.rope_neox, rs, dtype)
        self.scaling = qk ** -0.5
        if isinstance(rs, dict) and rs.get("factor"):
            m = yarn_get_mscale(rs["factor"], rs.get("mscale_all_dim", 0.0) or 0.0)
            self.scaling = self.scaling * m * m
        self.select_keys = None
        self.w_uk = None    # [heads, nope, kv_lora]
        self.w_uv = None    # [heads, kv_lora, v]

    def absorb(self):
        """Split kv_b_proj into the two per-head matrices of the absorbed form (after loading)."""
        w = self.kv_b_proj.weight.data.view(self.local_heads, self.nope + self.v_dim, self.kv_lora)
        self.w_uk = w[:, : self.nope, :].contiguous()
        self.w_uv = w[:, self.nope:, :].transpose(1, 2).contiguous()

    def forward(self, x, fb):
        T = x.shape[0]
        if self.w_uk is None:
            self.absorb()
        q_resid = None
        if self.q_lora:
            q_resid = self.q_a_layernorm(self.q_a_proj(x))
            q = self.q_b_proj(q_resid)
        else:
            q = self.q_proj(x)
        q = q.view(T, self.local_heads, self.nope + self.rope_dim)
        q_nope, q_pe = q[..., : self.nope], q[..., self.nope:]
        latent = self.kv_a_proj_with_mqa(x)
        kv_c = self.kv_a_layernorm(latent[:, : self.kv_lora].contiguous())
        k_pe = latent[:, self.kv_lora:].unsqueeze(1)
        if getattr(self, "skip_rope", False):          # position-free MLA (hybrids whose linear layers carry order)
            k_pe = k_pe.squeeze(1)
        else:
            cs = self.rotary_emb.cos_sin_cache
            q_pe = reference.apply_rope(q_pe, fb.positions, cs, self.rope_neox)
            k_pe = reference.apply_rope(k_pe, fb.positions, cs, self.rope_neox).squeeze(1)
        pool = fb.token_to_kv_pool
        pool.set_kv_buffer(self.layer_id, fb.out_cache_loc, kv_c, k_pe)
        # absorbed query: [T, h, nope] x [h, nope, r] -> [T, h, r]
        q_lat = torch.einsum("thn,hnr->thr", q_nope.float(), self.w_uk.float()).to(x.dtype)
        buf = pool.get_kv_buffer(self.layer_id)
        # sparse attention (an indexer picks the keys each query may see); None = dense
        allowed = self.select_keys(x, q_resid, fb) if self.select_keys is not None else None
        if fb.forward_mode.is_decode():
            o_lat = ops.mla_paged_attention(q_lat, q_pe.contiguous(), buf, fb.page_table, fb.req_pool_indices,
                                            fb.seq_lens, fb.page_size, self.scaling, self.kv_lora, allowed=allowed,
                                            max_seq_len=fb.max_seq_len)
        else:
            o_lat = ops.mla_paged_attention(q_lat, q_pe.contiguous(), buf, fb.page_table, fb.req_pool_indices,
                                            fb.seq_lens, fb.page_size, self.scaling, self.kv_lora, fb.cu_q_lens,
                                            fb.extend_prefix_lens, allowed=allowed)
        o = torch.einsum("thr,hrv->thv", o_lat.float(), self.w_uv.float()).to(x.dtype)
        return o.reshape(T, self.local_heads * self.v_dim)


class DeepseekMoE(nn.Module):
    def __init__(self, config, layer_id, dtype, correction_bias: bool | None = None):
        super().__init__()
        E = config.n_routed_experts
        bias = getattr(config, "topk_method", "greedy") == "noaux_tc" if correction_bias is None else correction_bias
        self.gate = GateLogit(config.hidden_size, E, dtype, correction_bias=bias,
                              score_func=getattr(config, "scoring_func", "softmax"))
        self.topk = TopK(config.num_experts_per_tok, renormalize=getattr(config, "norm_topk_prob", False),
                         num_expert_group=getattr(config, "n_group", 0) or 0,
                         topk_group=getattr(config, "topk_group", 0) or 0,
                         routed_scaling_factor=getattr(config, "routed_scaling_factor", 1.0),
                         scoring_func=getattr(config, "scoring_func", "softmax"))
        self.experts = FusedMoE(E, config.hidden_size, config.moe_intermediate_size, dtype, layer_id=layer_id)
        self.tp_size = self.experts.tp_size
        n_shared = getattr(config, "n_shared_experts", 0) or 0
        self.shared_experts = None
        if n_shared:
            self.shared_experts = DenseMLP(config.hidden_size, config.moe_intermediate_size * n_shared, dtype)
            self.shared_experts.down_proj.reduce_results = False

    def partial(self, x, out=None):
        w, ids = self.topk(self.gate(x), self.gate.e_score_correction_bias)
        add = self.shared_experts(x) if self.shared_experts is not None else None
        return self.experts(x, w, ids, add=add, out=out)


class DeepseekDecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype, attn_cls=None):
        super().__init__()
        eps = config.rms_norm_eps
        self.self_attn = (attn_cls or MLAAttention)(config, layer_id, dtype)
        first_dense = getattr(config, "first_k_dense_replace", 0)
        freq = getattr(config, "moe_layer_freq", 1) or 1
        self.is_sparse = (getattr(config, "n_routed_experts", None) is not None and layer_id >= first_dense
                          and layer_id % freq == 0)
        self.mlp = DeepseekMoE(config, layer_id, dtype) if self.is_sparse else \
            DenseMLP(config.hidden_size, config.intermediate_size, dtype)
        self.input_layernorm = RMSNorm(config.hidden_size, eps, dtype)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps, dtype)

    def forward(self, h_normed, residual, fb, next_norm):
        a = self.self_attn(h_normed, fb)
        h, residual = row_linear_add_norm(self.self_attn.o_proj, a, residual, self.post_attention_layernorm)
        if self.is_sparse:
            return partial_add_norm(lambda out: self.mlp.partial(h, out), h.shape[0], h.shape[1], residual, next_norm,
                                    self.mlp.tp_size, block=self.mlp, x=h)
        act = self.mlp.act_fn(self.mlp.gate_up_proj(h))
        return row_linear_add_norm(self.mlp.down_proj, act, residual, next_norm)


class DeepseekModel(nn.Module):
    def __init__(self, config, dtype, attn_cls=None):
        super().__init__()
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        self.layers = nn.ModuleList([DeepseekDecoderLayer(config, i, dtype, attn_cls)
                                     for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps, dtype)

    def forward(self, input_ids, fb, input_embeds=None):
        residual = self.embed_tokens(input_ids) if input_embeds is None else input_embeds
        h = self.layers[0].input_layernorm(residual)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].input_layernorm if i + 1 < n else self.norm
            h, residual = layer(h, residual, fb, nxt)
        return h


class DeepseekV3ForCausalLM(nn.Module):
    stacked = [(".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1)]
    optional_params = {"e_score_correction_bias"}
    attn_cls = None

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        self.config = config
        self.dtype = dtype
        self.model = DeepseekModel(config, dtype, self.attn_cls)
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        self.logits_processor = LogitsProcessor(config.vocab_size)

    def forward(self, input_ids, fb, input_embeds=None):
        return self.logits_processor(self.model(input_ids, fb, input_embeds), self.lm_head, fb)

    def load_weights(self, weights):
        params = dict(self.named_parameters())
        modules = dict(self.named_modules())
        loaded = set()
        n_layers = self.config.num_hidden_layers
        for name, w in weights:
            if "rotary_emb" in name or name.endswith("_scale_inv") and False:
                continue
            if name.startswith("model.layers."):
                if int(name.split(".")[2]) >= n_layers:
                    continue        # multi-token-prediction head layers are loaded by the draft model
            if name == "lm_head.weight" and self.tie:
                continue
            if ".mlp.experts." in name and name.endswith(".weight"):
                head, tail = name.split(".mlp.experts.")
                e_str, proj, _ = tail.split(".")
                shard = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down"}[proj]
                pname = f"{head}.mlp.experts." + ("w2_weight" if shard == "down" else "w13_weight")
                if pname in params:
                    p = params[pname]
                    modules[f"{head}.mlp.experts"].weight_loader(p, w, shard, int(e_str))
                    loaded.add(pname)
                continue
            if name.endswith(".mlp.experts.gate_up_proj") or name.endswith(".mlp.experts.down_proj"):
                head = name.rsplit(".mlp.experts.", 1)[0]
                mod = modules[f"{head}.mlp.experts"]
                if name.endswith("gate_up_proj"):
                    p = params[f"{head}.mlp.experts.w13_weight"]
                    I = w.shape[1] // 2
                    for e in range(w.shape[0]):
                        mod.weight_loader(p, w[e, :I], "gate", e)
                        mod.weight_loader(p, w[e, I:], "up", e)
                    loaded.add(f"{head}.mlp.experts.w13_weight")
                else:
                    p = params[f"{head}.mlp.experts.w2_weight"]
                    for e in range(w.shape[0]):
                        mod.weight_loader(p, w[e], "down", e)
                    loaded.add(f"{head}.mlp.experts.w2_weight")
                continue
            target, shard = name, None
            if ".mlp.gate.e_score_correction_bias" in name:
                p = params.get(name)
                if p is not None:
                    p.data.copy_(w.float())
                    loaded.add(name)
                continue
            for pfrag, cfrag, sid in self.stacked:
                if cfrag in name and ".experts." not in name:
                    target, shard = name.replace(cfrag, pfrag), sid
                    break
            if target not in params:
                continue
            mod = modules[target.rsplit(".", 1)[0]]
            p = params[target]
            mod.weight_loader(p, w.to(p.dtype) if w.dtype != p.dtype else w, shard)
            loaded.add(target)
        self.post_load_weights()
        return loaded

    def post_load_weights(self):
        if self.tie:
            self.lm_head.tie_to(self.model.embed_tokens)
        for layer in self.model.layers:
            layer.self_attn.absorb()


class DeepseekV2ForCausalLM(DeepseekV3ForCausalLM):
    pass


class KimiK2ForCausalLM(DeepseekV3ForCausalLM):
    pass


EntryClass = [DeepseekV3ForCausalLM, DeepseekV2ForCausalLM, KimiK2ForCausalLM]
