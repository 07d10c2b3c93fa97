"""Qwen3-Next / Qwen3.5 hybrid decoders (reference `python/sgl_jax/srt/models/qwen3_5.py`):
three of every four layers mix tokens with a Gated DeltaNet (linear attention over a recurrent
state), the fourth with gated softmax attention (output multiplied by `sigmoid(gate)`, q/k
RMSNorm, rotary on a quarter of the head); norms are zero-centred (`1 + w`); the FFN is a
softmax-routed MoE with a sigmoid-gated shared expert, or dense."""

from __future__ import annotations

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding, get_rope
from ..layers.layernorm import GemmaRMSNorm
from ..layers.linear import ColumnParallelLinear, RowParallelLinear
from ..layers.linear_attention import GatedDeltaNet
from ..layers.logits_processor import LogitsProcessor
from ..layers.radix_attention import RadixAttention
from ..parallel import state as ps
from .llama import DenseMLP, LlamaForCausalLM
from .moe_loading import load_sparse_weights
from .qwen3_moe import SparseMoeBlock


class GatedAttention(nn.Module):
    def __init__(self, config, kv_layer_id, dtype):
        super().__init__()
        H = config.hidden_size
        self.head_dim = config.head_dim
        nh, nkv = config.num_attention_heads, config.num_key_value_heads
        tp = ps.tp_size()
        assert nh % tp == 0 and nkv % tp == 0, "hybrid attention layers need tp <= num_key_value_heads"
        self.nh, self.nkv = nh // tp, nkv // tp
        bias = getattr(config, "attention_bias", False)
        self.q_proj = ColumnParallelLinear(H, nh * self.head_dim * 2, bias, dtype)       # per head: [q | gate]
        self.k_proj = ColumnParallelLinear(H, nkv * self.head_dim, bias, dtype)
        self.v_proj = ColumnParallelLinear(H, nkv * self.head_dim, bias, dtype)
        self.o_proj = RowParallelLinear(nh * self.head_dim, H, bias, dtype)
        eps = config.rms_norm_eps
        self.q_norm = GemmaRMSNorm(self.head_dim, eps, dtype)
        self.k_norm = GemmaRMSNorm(self.head_dim, eps, dtype)
        rp = getattr(config, "rope_parameters", None) or {}
        theta = getattr(config, "rope_theta", None) or rp.get("rope_theta", 10000.0)
        prf = getattr(config, "partial_rotary_factor", None) or rp.get("partial_rotary_factor", 1.0)
        self.rotary_emb = get_rope(self.head_dim, int(self.head_dim * prf), config.max_position_embeddings, theta,
                                   True, None, dtype)
        self.attn = RadixAttention(self.nh, self.head_dim, self.head_dim ** -0.5, self.nkv, kv_layer_id)

    def forward(self, x, fb):
        T = x.shape[0]
        qg = self.q_proj(x).view(T, self.nh, 2 * self.head_dim)
        q, gate = qg[..., : self.head_dim], qg[..., self.head_dim:]
        qkv = torch.cat([q.reshape(T, -1), self.k_proj(x), self.v_proj(x)], dim=-1)
        o = self.attn(qkv, fb, self.rotary_emb, self.q_norm, self.k_norm, gemma_norm=True)
        o = o * torch.sigmoid(gate.reshape(T, -1).float()).to(o.dtype)
        return self.o_proj(o)


class Qwen3NextDecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype, kv_layer_id, linear_index):
        super().__init__()
        eps = config.rms_norm_eps
        self.layer_type = config.layer_types[layer_id]
        if self.layer_type == "linear_attention":
            self.linear_attn = GatedDeltaNet(config, linear_index, dtype)
        else:
            self.self_attn = GatedAttention(config, kv_layer_id, dtype)
        mlp_only = set(getattr(config, "mlp_only_layers", None) or [])
        step = getattr(config, "decoder_sparse_step", 1) or 1
        n_exp = getattr(config, "num_experts", 0) or 0
        self.is_sparse = layer_id not in mlp_only and n_exp > 0 and (layer_id + 1) % step == 0
        self.mlp = SparseMoeBlock(config, layer_id, dtype, shared_expert=True) if self.is_sparse else \
            DenseMLP(config.hidden_size, config.intermediate_size, dtype)
        self.input_layernorm = GemmaRMSNorm(config.hidden_size, eps, dtype)
        self.post_attention_layernorm = GemmaRMSNorm(config.hidden_size, eps, dtype)

    def forward(self, x, fb):
        h = self.input_layernorm(x)
        h = self.linear_attn(h, fb) if self.layer_type == "linear_attention" else self.self_attn(h, fb)
        x = x + h
        h = self.post_attention_layernorm(x)
        if self.is_sparse:
            y = self.mlp.partial(h)
            if self.mlp.tp_size > 1:
                y = ps.all_reduce(y)
        else:
            y = self.mlp(h)
        return x + y


class Qwen3NextModel(nn.Module):
    def __init__(self, config, dtype):
        super().__init__()
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        layers, kv_id, lin_id = [], 0, 0
        for i, t in enumerate(config.layer_types):
            layers.append(Qwen3NextDecoderLayer(config, i, dtype, kv_id, lin_id))
            if t == "linear_attention":
                lin_id += 1
            else:
                kv_id += 1
        self.layers = nn.ModuleList(layers)
        self.num_kv_layers, self.num_linear_layers = kv_id, lin_id
        self.norm = GemmaRMSNorm(config.hidden_size, config.rms_norm_eps, dtype)

    def forward(self, input_ids, fb, input_embeds=None):
        x = self.embed_tokens(input_ids) if input_embeds is None else input_embeds
        for layer in self.layers:
            x = layer(x, fb)
        return self.norm(x)


class Qwen3NextForCausalLM(LlamaForCausalLM):
    is_hybrid_linear = True

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        config = getattr(config, "text_config", None) or config
        if not getattr(config, "layer_types", None):
            k = getattr(config, "full_attention_interval", 4)
            config.layer_types = ["full_attention" if (i + 1) % k == 0 else "linear_attention"
                                  for i in range(config.num_hidden_layers)]
        self.config = config
        self.dtype = dtype
        self.model = Qwen3NextModel(config, dtype)
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        self.logits_processor = LogitsProcessor(config.vocab_size)
        self.capture_aux_hidden_states = False
        self.num_kv_layers = self.model.num_kv_layers
        gdn = next(l.linear_attn for l in self.model.layers if l.layer_type == "linear_attention")
        # what the runner needs to size the recurrent state pool
        self.recurrent_spec = dict(num_layers=self.model.num_linear_layers, conv_dim=gdn.conv_dim,
                                   conv_kernel=gdn.conv_kernel, num_heads=gdn.nv, head_k_dim=gdn.dk, head_v_dim=gdn.dv)

    def forward(self, input_ids, fb, input_embeds=None):
        return self.logits_processor(self.model(input_ids, fb, input_embeds), self.lm_head, fb)

    def load_weights(self, weights):
        return load_sparse_weights(
            self, weights, renames=[(".linear_attn.conv1d.weight", ".linear_attn.conv1d_weight"),
                                    ("model.language_model.", "model.")],
            skip=("mtp.", "visual."), stacked=[(".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1)])


def fuse_split_gdn_projections(weights, config):
    """Qwen3.5 checkpoints store the Gated DeltaNet input projection as four tensors (`in_proj_qkv` with all query
    heads, then all key heads, then all value heads; `in_proj_z`; `in_proj_b`; `in_proj_a`), Qwen3-Next as two
    tensors grouped per key head (`in_proj_qkvz`: q, k, the group's values, the group's gates; `in_proj_ba`).  The
    layer keeps the grouped layout (one GEMM each); this regroups the rows of a Qwen3.5 checkpoint while it streams
    by (reference `models/qwen3_5.py` `_create_qwen3_5_weight_mappings`, the fused targets of the four HF keys)."""
    nk, nv = config.linear_num_key_heads, config.linear_num_value_heads
    dk, dv = config.linear_key_head_dim, config.linear_value_head_dim
    r, key_dim = nv // nk, nk * dk
    parts = ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a")
    pending: dict[str, dict[str, torch.Tensor]] = {}
    for name, w in weights:
        hit = next((p for p in parts if name.endswith(f".linear_attn.{p}.weight")), None)
        if hit is None:
            yield name, w
            continue
        prefix = name[: -len(f"{hit}.weight")]
        got = pending.setdefault(prefix, {})
        got[hit] = w
        if len(got) < 4:
            continue
        pending.pop(prefix)
        qkv, z, b, a = (got[p] for p in parts)
        H = qkv.shape[1]
        q = qkv[:key_dim].reshape(nk, dk, H)
        k = qkv[key_dim:2 * key_dim].reshape(nk, dk, H)
        v = qkv[2 * key_dim:].reshape(nk, r * dv, H)
        yield prefix + "in_proj_qkvz.weight", torch.cat([q, k, v, z.reshape(nk, r * dv, H)], 1).reshape(-1, H)
        yield prefix + "in_proj_ba.weight", torch.cat([b.reshape(nk, r, H), a.reshape(nk, r, H)], 1).reshape(-1, H)
    if pending:
        raise RuntimeError(f"incomplete Gated DeltaNet projections in the checkpoint: {sorted(pending)[:3]}")


class Qwen3_5ForCausalLM(Qwen3NextForCausalLM):
    """Qwen3.5 text model (dense); also the text part of `Qwen3_5ForConditionalGeneration` checkpoints, whose vision
    tower and multi-token-prediction head are skipped like in the reference."""

    def load_weights(self, weights):
        return super().load_weights(fuse_split_gdn_projections(weights, self.config))


class Qwen3_5MoeForCausalLM(Qwen3_5ForCausalLM):
    pass


class Qwen3_5ForConditionalGeneration(Qwen3_5ForCausalLM):
    pass


class Qwen3_5MoeForConditionalGeneration(Qwen3_5ForCausalLM):
    pass


EntryClass = [Qwen3NextForCausalLM, Qwen3_5ForCausalLM, Qwen3_5MoeForCausalLM, Qwen3_5ForConditionalGeneration,
              Qwen3_5MoeForConditionalGeneration]
