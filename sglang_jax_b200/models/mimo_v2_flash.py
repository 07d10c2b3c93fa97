"""MiMo-V2-Flash / MiMo-V2-Pro (reference `python/sgl_jax/srt/models/mimo_v2_flash.py`,
`mimo_v2_pro.py`): layers follow `hybrid_layer_pattern` — sliding-window layers with their own
head count / head sizes and a learned attention-sink bias, full-attention layers otherwise; the
value head may be narrower than the key head (it is zero-padded inside the KV cache); FFNs follow
`moe_layer_freq` (sigmoid routing with correction bias, no shared expert)."""

from __future__ import annotations

import torch
from torch import nn

from ..layers.embeddings import ParallelLMHead, VocabParallelEmbedding, get_rope
from ..layers.layernorm import RMSNorm
from ..layers.linear import QKVParallelLinear, RowParallelLinear
from ..layers.logits_processor import LogitsProcessor
from ..layers.radix_attention import RadixAttention
from ..parallel import state as ps
from .deepseek_v3 import DeepseekMoE
from .llama import DenseMLP, LlamaForCausalLM
from .moe_loading import load_sparse_weights


def _is_swa(config, i: int) -> bool:
    pat = getattr(config, "hybrid_layer_pattern", None)
    return bool(pat is not None and 0 <= i < len(pat) and pat[i] == 1)


def _is_moe(config, i: int) -> bool:
    f = getattr(config, "moe_layer_freq", None)
    return bool(f is not None and not isinstance(f, int) and 0 <= i < len(f) and f[i])


class MiMoV2Attention(nn.Module):
    def __init__(self, config, layer_id, dtype, swa: bool):
        super().__init__()
        H = config.hidden_size
        if swa:
            nh, nkv = config.swa_num_attention_heads, config.swa_num_key_value_heads
            hd, vd = config.swa_head_dim, getattr(config, "swa_v_head_dim", None) or config.swa_head_dim
            theta = getattr(config, "swa_rope_theta", None) or getattr(config, "rope_theta", 1e6)
            window = getattr(config, "sliding_window_size", None) or getattr(config, "sliding_window", 0) or 0
            sink = bool(getattr(config, "add_swa_attention_sink_bias", False))
        else:
            nh, nkv = config.num_attention_heads, config.num_key_value_heads
            hd, vd = config.head_dim, getattr(config, "v_head_dim", None) or config.head_dim
            theta = getattr(config, "rope_theta", 1e6)
            window = 0
            sink = bool(getattr(config, "add_full_attention_sink_bias", False))
        self.hd, self.vd = hd, vd
        self.qkv_proj = QKVParallelLinear(H, hd, nh, nkv, getattr(config, "attention_bias", False), dtype, v_head_dim=vd)
        self.o_proj = RowParallelLinear(nh * vd, H, False, dtype)
        prf = getattr(config, "partial_rotary_factor", 1.0)
        self.rotary_emb = get_rope(hd, int(hd * prf), config.max_position_embeddings, theta, True,
                                   getattr(config, "rope_scaling", None), dtype)
        self.value_scale = getattr(config, "attention_value_scale", None)
        self.attn = RadixAttention(self.qkv_proj.num_heads, hd, hd ** -0.5, self.qkv_proj.num_kv_heads, layer_id, window)
        self.attention_sink_bias = nn.Parameter(torch.zeros(self.qkv_proj.num_heads, dtype=torch.float32),
                                                requires_grad=False) if sink else None
        self._sink_rank = self.qkv_proj.tp_rank

    def weight_loader(self, param, w, shard_id=None):      # the sink bias is sharded with the query heads
        n = param.shape[0]
        param.data.copy_(w.float().narrow(0, self._sink_rank * n, n))

    def forward(self, x, fb):
        qp = self.qkv_proj
        qkv = qp(x)
        if self.vd != self.hd or self.value_scale is not None:
            q, k, v = qkv.split([qp.q_size, qp.k_size, qp.v_size], dim=-1)
            if self.value_scale is not None:
                v = v * self.value_scale
            if self.vd != self.hd:       # the cache stores V at key width
                v = torch.nn.functional.pad(v.view(-1, qp.num_kv_heads, self.vd), (0, self.hd - self.vd)).flatten(1)
            qkv = torch.cat([q, k, v], dim=-1)
        o = self.attn(qkv, fb, self.rotary_emb, sinks=self.attention_sink_bias)
        if self.vd != self.hd:
            o = o.view(-1, qp.num_heads, self.hd)[..., : self.vd].reshape(-1, qp.num_heads * self.vd)
        return self.o_proj(o)


class MiMoV2DecoderLayer(nn.Module):
    def __init__(self, config, layer_id, dtype):
        super().__init__()
        self.is_swa = _is_swa(config, layer_id)
        self.self_attn = MiMoV2Attention(config, layer_id, dtype, self.is_swa)
        self.is_sparse = _is_moe(config, layer_id)
        self.mlp = DeepseekMoE(config, layer_id, dtype) if self.is_sparse else \
            DenseMLP(config.hidden_size, config.intermediate_size, dtype)
        eps = getattr(config, "layernorm_epsilon", None) or getattr(config, "rms_norm_eps", 1e-6)
        self.input_layernorm = RMSNorm(config.hidden_size, eps, dtype)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps, dtype)

    def forward(self, x, fb):
        x = x + self.self_attn(self.input_layernorm(x), fb)
        h = self.post_attention_layernorm(x)
        if self.is_sparse:
            y = self.mlp.partial(h)
            if self.mlp.tp_size > 1:
                y = ps.all_reduce(y)
        else:
            y = self.mlp(h)
        return x + y


class MiMoV2FlashForCausalLM(LlamaForCausalLM):
    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        nn.Module.__init__(self)
        if not hasattr(config, "n_routed_experts"):
            config.n_routed_experts = getattr(config, "num_experts", 0)
        if not hasattr(config, "n_shared_experts"):
            config.n_shared_experts = 0
        self.config, self.dtype = config, dtype
        model = nn.Module()
        model.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, dtype)
        model.layers = nn.ModuleList([MiMoV2DecoderLayer(config, i, dtype) for i in range(config.num_hidden_layers)])
        eps = getattr(config, "layernorm_epsilon", None) or getattr(config, "rms_norm_eps", 1e-6)
        model.norm = RMSNorm(config.hidden_size, eps, dtype)
        self.model = model
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size, dtype)
        self.tie = bool(getattr(config, "tie_word_embeddings", False))
        self.logits_processor = LogitsProcessor(config.vocab_size)
        self.capture_aux_hidden_states = False
        swa = [i for i in range(config.num_hidden_layers) if _is_swa(config, i)]
        if swa and len(swa) < config.num_hidden_layers:
            self.swa_layer_ids = swa
            tp = ps.tp_size()
            self.swa_kv_shape = (max(1, config.swa_num_key_value_heads // tp), config.swa_head_dim)

    def forward(self, input_ids, fb, input_embeds=None):
        x = self.model.embed_tokens(input_ids) if input_embeds is None else input_embeds
        for layer in self.model.layers:
            x = layer(x, fb)
        return self.logits_processor(self.model.norm(x), self.lm_head, fb)

    def load_weights(self, weights):
        loaded = load_sparse_weights(self, weights, max_layer=self.config.num_hidden_layers, skip=("mtp.",))
        return loaded


def infer_qkv_shards(rows: int, scale_rows: int, nh: int, nkv: int, hd: int, vd: int, block: int) -> tuple[int, int]:
    """`(shards, kv_heads)` of a fused QKV tensor that was block-quantised shard by shard: the shard count (largest
    first, a smaller one can satisfy the sizes too but splits Q / K / V in the wrong places) and the number of KV
    heads the checkpoint really holds (the config may list a replicated count) for which `shards` blocks of
    `ceil(per_shard / block)` scale rows and `per_shard` weight rows add up to what the checkpoint has."""
    for kv in sorted((d for d in range(1, nkv + 1) if nkv % d == 0), reverse=True):
        for tp in sorted((d for d in range(1, nh + 1) if nh % d == 0), reverse=True):
            if kv % tp:
                continue
            per = (nh // tp) * hd + (kv // tp) * (hd + vd)
            if per * tp == rows and -(-per // block) * tp == scale_rows:
                return tp, kv
    raise ValueError(f"cannot infer how the fused QKV was sharded: rows={rows} scale_rows={scale_rows} heads={nh} "
                     f"kv_heads={nkv} head_dim={hd} v_head_dim={vd} block={block}")


class MiMoV2ProForCausalLM(MiMoV2FlashForCausalLM):
    """MiMo-V2-Pro (reference `python/sgl_jax/srt/models/mimo_v2_pro.py`): the Flash architecture with the attention
    input projection stored fused as `self_attn.qkv_proj`.  In bf16 checkpoints its rows are `[Q | K | V]`.  In the
    block-FP8 release the tensor was quantised per tensor-parallel shard and the shards concatenated
    (`[Q0 K0 V0 | Q1 K1 V1 | ...]`, each shard with its own `ceil(rows / 128)` scale rows, so a scale block can
    straddle a K / V border inside a shard but never a shard border): every shard is de-quantised on its own grid
    and its Q / K / V rows are regrouped; the attention projections then hold bf16 weights like in the reference
    (`utils/weight_utils.py` `dequant_fused_qkv`)."""

    def preprocess_checkpoint(self, weights):
        cfg = self.config
        qc = getattr(cfg, "quantization_config", None) or {}
        wbs = qc.get("weight_block_size") if isinstance(qc, dict) else getattr(qc, "weight_block_size", None)
        block = int(wbs[0]) if wbs else 128
        fp8 = (torch.float8_e4m3fn, torch.float8_e5m2)
        pending: dict[str, dict[str, torch.Tensor]] = {}

        def dims(prefix: str):
            i = int(prefix.split("layers.")[1].split(".")[0])
            if _is_swa(cfg, i):
                return (cfg.swa_num_attention_heads, cfg.swa_num_key_value_heads, cfg.swa_head_dim,
                        getattr(cfg, "swa_v_head_dim", None) or cfg.swa_head_dim)
            return (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                    getattr(cfg, "v_head_dim", None) or cfg.head_dim)

        def emit(prefix, q, k, v):
            yield prefix + "q_proj.weight", q
            yield prefix + "k_proj.weight", k
            yield prefix + "v_proj.weight", v

        for name, w in weights:
            if ".self_attn.qkv_proj." not in name:
                yield name, w
                continue
            prefix, leaf = name.split("qkv_proj.")
            nh, nkv, hd, vd = dims(prefix)
            if leaf == "weight" and w.dtype not in fp8:
                kv = (w.shape[0] - nh * hd) // (hd + vd)                   # KV heads the checkpoint really holds
                q, k, v = torch.split(w, [nh * hd, kv * hd, kv * vd], 0)
                yield from emit(prefix, q, k, v)
                continue
            got = pending.setdefault(prefix, {})
            got["scale" if leaf.startswith("weight_scale") else "weight"] = w
            if len(got) < 2:
                continue
            pending.pop(prefix)
            wq, sc = got["weight"], got["scale"].float()
            tp, kv = infer_qkv_shards(wq.shape[0], sc.shape[0], nh, nkv, hd, vd, block)
            pq, pk, pv = (nh // tp) * hd, (kv // tp) * hd, (kv // tp) * vd
            per, nb = pq + pk + pv, -(-(pq + pk + pv) // block)
            parts = ([], [], [])
            for s in range(tp):
                rows = wq[s * per:(s + 1) * per].float()
                rs = sc[s * nb:(s + 1) * nb].repeat_interleave(block, 0)[:per].repeat_interleave(block, 1)
                for dst, piece in zip(parts, torch.split(rows * rs[:, : rows.shape[1]], [pq, pk, pv], 0)):
                    dst.append(piece)
            yield from emit(prefix, *(torch.cat(p, 0).to(self.dtype) for p in parts))
        if pending:
            raise RuntimeError(f"fused QKV without its scale (or the reverse): {sorted(pending)[:3]}")


class MiMoV2ForCausalLM(MiMoV2ProForCausalLM):
    """The architecture string MiMo-V2-Pro checkpoints carry."""


EntryClass = [MiMoV2FlashForCausalLM, MiMoV2ProForCausalLM, MiMoV2ForCausalLM]
