"""Qwen3-MoE / Qwen2-MoE sparse decoders (reference `python/sgl_jax/srt/models/qwen3_moe.py`,
`qwen2_moe.py`): Qwen3 attention, every `decoder_sparse_step`-th layer (not in `mlp_only_layers`)
replaces the MLP with softmax top-k routed experts (Qwen2-MoE adds a sigmoid-gated shared expert)."""

from __future__ import annotations

import torch
from torch import nn

from ..layers.fused_block import partial_add_norm, row_linear_add_norm
from ..layers.gate import GateLogit, TopK
from ..layers.layernorm import RMSNorm
from ..layers.linear import ReplicatedLinear
from ..layers.moe import FusedMoE
from ..parallel import state as ps
from .llama import DenseAttention, DenseMLP, DenseModel, LlamaForCausalLM


class SparseMoeBlock(nn.Module):
    def __init__(self, config, layer_id, dtype, shared_expert: bool = False):
        super().__init__()
        self.hidden = config.hidden_size
        self.gate = GateLogit(config.hidden_size, config.num_experts, dtype)
        self.topk = TopK(config.num_experts_per_tok, renormalize=getattr(config, "norm_topk_prob", True))
        self.experts = FusedMoE(config.num_experts, config.hidden_size, config.moe_intermediate_size, dtype,
                                layer_id=layer_id)
        self.tp_size = self.experts.tp_size
        self.shared_expert = None
        if shared_expert and getattr(config, "shared_expert_intermediate_size", 0):
            self.shared_expert = DenseMLP(config.hidden_size, config.shared_expert_intermediate_size, dtype)
            self.shared_expert.down_proj.reduce_results = False
            self.shared_expert_gate = ReplicatedLinear(config.hidden_size, 1, False, dtype)

    def partial(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        logits = self.gate(x)
        w, ids = self.topk(logits)
        add = None
        if self.shared_expert is not None:
            s = self.shared_expert(x)
            add = (torch.sigmoid(self.shared_expert_gate(x).float()) * s.float()).to(x.dtype)
            if self.tp_size > 1 and self.experts.expert_parallel is False:
                pass   # both partials are slices of the same reduction
        return self.experts(x, w, ids, add=add, out=out)


class Qwen3MoeDecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype, **attn_kw):
        super().__init__()
        eps = getattr(config, "rms_norm_eps", 1e-6)
        self.self_attn = DenseAttention(config, layer_id, dtype, **attn_kw)
        mlp_only = set(getattr(config, "mlp_only_layers", None) or [])
        step = getattr(config, "decoder_sparse_step", 1) or 1
        self.is_sparse = layer_id not in mlp_only and config.num_experts > 0 and (layer_id + 1) % step == 0
        if self.is_sparse:
            self.mlp = SparseMoeBlock(config, layer_id, dtype, shared_expert=attn_kw.get("qkv_bias", False))
        else:
            self.mlp = DenseMLP(config.hidden_size, config.intermediate_size, dtype)
        self.input_layernorm = RMSNorm(config.hidden_size, eps, dtype)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps, dtype)

    def forward(self, hidden_normed, residual, forward_batch, next_norm):
        attn_out = self.self_attn(hidden_normed, forward_batch)
        h, residual = row_linear_add_norm(self.self_attn.o_proj, attn_out, residual, self.post_attention_layernorm)
        if self.is_sparse:
            return partial_add_norm(lambda out: self.mlp.partial(h, out), h.shape[0], h.shape[1], residual, next_norm,
                                    self.mlp.tp_size, block=self.mlp, x=h)
        act = self.mlp.act_fn(self.mlp.gate_up_proj(h))
        return row_linear_add_norm(self.mlp.down_proj, act, residual, next_norm)


class Qwen3MoeModel(DenseModel):
    layer_cls = Qwen3MoeDecoderLayer


class Qwen3MoeForCausalLM(LlamaForCausalLM):
    model_cls = Qwen3MoeModel

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        from ..layers.embeddings import ParallelLMHead
        from ..layers.logits_processor import LogitsProcessor
        self.config = config
        self.dtype = dtype
        self.model = self.model_cls(config, dtype, **self._attn_kw(config))
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        self.logits_processor = LogitsProcessor(config.vocab_size)
        self.capture_aux_hidden_states = False

    def _attn_kw(self, config):
        return dict(qkv_bias=getattr(config, "attention_bias", False), o_bias=False, qk_norm=True)

    def load_weights(self, weights):
        params = dict(self.named_parameters())
        modules = dict(self.named_modules())

        def rest():
            for name, w in weights:
                if ".mlp.experts." in name and name.endswith(".weight"):
                    # model.layers.{i}.mlp.experts.{e}.{gate|up|down}_proj.weight
                    head, tail = name.split(".mlp.experts.")
                    e_str, proj, _ = tail.split(".")
                    shard = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down"}[proj]
                    pname = f"{head}.mlp.experts." + ("w2_weight" if shard == "down" else "w13_weight")
                    if pname in params:
                        p = params[pname]
                        modules[f"{head}.mlp.experts"].weight_loader(p, w, shard, int(e_str))
                        self._loaded_extra.add(pname)
                    continue
                if name.endswith(".mlp.experts.gate_up_proj") or name.endswith(".mlp.experts.down_proj"):
                    # fused layout: [E, 2I, H] (gate rows then up rows) / [E, H, I]
                    head = name.rsplit(".mlp.experts.", 1)[0]
                    mod = modules[f"{head}.mlp.experts"]
                    if name.endswith("gate_up_proj"):
                        p = params[f"{head}.mlp.experts.w13_weight"]
                        I = w.shape[1] // 2
                        for e in range(w.shape[0]):
                            mod.weight_loader(p, w[e, :I], "gate", e)
                            mod.weight_loader(p, w[e, I:], "up", e)
                        self._loaded_extra.add(f"{head}.mlp.experts.w13_weight")
                    else:
                        p = params[f"{head}.mlp.experts.w2_weight"]
                        for e in range(w.shape[0]):
                            mod.weight_loader(p, w[e], "down", e)
                        self._loaded_extra.add(f"{head}.mlp.experts.w2_weight")
                    continue
                yield name, w
        self._loaded_extra = set()
        loaded = super().load_weights(rest())
        return loaded | self._loaded_extra


class Qwen2MoeForCausalLM(Qwen3MoeForCausalLM):
    def _attn_kw(self, config):
        return dict(qkv_bias=True, o_bias=False, qk_norm=False)


EntryClass = [Qwen3MoeForCausalLM, Qwen2MoeForCausalLM]
