"""UMT5 / T5 (reference `python/sgl_jax/srt/models/umt5.py`, `multimodal/models/t5`): the text encoder that
prompts the Wan video pipeline, and the decoder / encoder-decoder / conditional-generation classes of the same
checkpoint family (`UMT5DecoderModel`, `UMT5Model`, `UMT5ForConditionalGeneration`).  Unscaled dot-product attention
with a learned relative-position bias (one table per layer in UMT5, shared from layer 0 in T5; bidirectional buckets
in the encoder, one-sided in the decoder, none in cross-attention), gated-GELU FFN, RMS layer norm without mean
subtraction.  `UMT5ForConditionalGeneration.generate` decodes greedily with cached self-attention keys / values and
cross-attention keys / values projected once per prompt."""

from __future__ import annotations

import math
from typing import Iterable

import torch
from torch import nn

from .. import ops


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def relative_position_bucket(rel: torch.Tensor, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Bidirectional T5 bucketing of `key_pos - query_pos`."""
    nb = num_buckets // 2
    out = (rel > 0).long() * nb
    rel = rel.abs()
    max_exact = nb // 2
    small = rel < max_exact
    large = max_exact + (torch.log(rel.float().clamp_min(1) / max_exact) / math.log(max_distance / max_exact)
                         * (nb - max_exact)).long()
    large = torch.minimum(large, torch.full_like(large, nb - 1))
    return out + torch.where(small, rel, large)


class T5Block(nn.Module):
    def __init__(self, cfg, dtype, has_bias_table: bool):
        super().__init__()
        D, H, dk, F = cfg.d_model, cfg.num_heads, cfg.d_kv, cfg.d_ff
        self.H, self.dk = H, dk
        mk = lambda o, i: nn.Parameter(torch.empty(o, i, dtype=dtype), requires_grad=False)
        self.q, self.k, self.v, self.o = mk(H * dk, D), mk(H * dk, D), mk(H * dk, D), mk(D, H * dk)
        self.rel_bias = nn.Parameter(torch.empty(cfg.relative_attention_num_buckets, H, dtype=dtype),
                                     requires_grad=False) if has_bias_table else None
        self.ln0 = nn.Parameter(torch.ones(D, dtype=dtype), requires_grad=False)
        self.ln1 = nn.Parameter(torch.ones(D, dtype=dtype), requires_grad=False)
        self.gated = bool(getattr(cfg, "is_gated_act", True))
        self.wi_0 = mk(F, D)
        self.wi_1 = mk(F, D) if self.gated else None
        self.wo = mk(D, F)
        act = getattr(cfg, "dense_act_fn", "gelu_new")
        self.act = (lambda t: torch.nn.functional.gelu(t, approximate="tanh")) if "gelu" in act else torch.relu
        self.eps = cfg.layer_norm_epsilon

    def forward(self, x, bias, key_mask):
        B, T, D = x.shape
        h = _rms(x, self.ln0, self.eps).reshape(B * T, D)
        q = ops.linear(h, self.q).view(B, T, self.H, self.dk).transpose(1, 2)
        k = ops.linear(h, self.k).view(B, T, self.H, self.dk).transpose(1, 2)
        v = ops.linear(h, self.v).view(B, T, self.H, self.dk).transpose(1, 2)
        s = torch.matmul(q.float(), k.float().transpose(-1, -2)) + bias          # T5 does not scale by sqrt(d)
        if key_mask is not None:
            s = s.masked_fill(~key_mask[:, None, None, :], float("-inf"))
        a = torch.matmul(torch.softmax(s, -1), v.float()).to(x.dtype).transpose(1, 2).reshape(B * T, self.H * self.dk)
        x = x + ops.linear(a, self.o).view(B, T, D)
        h = _rms(x, self.ln1, self.eps).reshape(B * T, D)
        g = self.act(ops.linear(h, self.wi_0))
        if self.gated:
            g = g * ops.linear(h, self.wi_1)
        return x + ops.linear(g, self.wo).view(B, T, D)


class UMT5EncoderModel(nn.Module):
    per_layer_bias = True

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        self.config = config
        self.shared = nn.Parameter(torch.empty(config.vocab_size, config.d_model, dtype=dtype), requires_grad=False)
        self.blocks = nn.ModuleList([T5Block(config, dtype, self.per_layer_bias or i == 0)
                                     for i in range(config.num_layers)])
        self.final_ln = nn.Parameter(torch.ones(config.d_model, dtype=dtype), requires_grad=False)

    @torch.inference_mode()
    def encode(self, input_ids: torch.Tensor, attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        """`input_ids [B, T]` -> last hidden state `[B, T, d_model]`."""
        B, T = input_ids.shape
        x = self.shared[input_ids]
        pos = torch.arange(T, device=input_ids.device)
        buckets = relative_position_bucket(pos[None, :] - pos[:, None], self.config.relative_attention_num_buckets,
                                           self.config.relative_attention_max_distance)
        mask = attention_mask.bool() if attention_mask is not None else None
        bias = None
        for blk in self.blocks:
            if blk.rel_bias is not None:
                bias = blk.rel_bias[buckets].permute(2, 0, 1).unsqueeze(0).float()     # [1, H, T, T]
            x = blk(x, bias, mask)
        return _rms(x, self.final_ln, self.config.layer_norm_epsilon)

    forward = encode

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        table = {"shared.weight": "shared", "encoder.embed_tokens.weight": "shared",
                 "encoder.final_layer_norm.weight": "final_ln"}
        sub = {"layer.0.SelfAttention.q.weight": "q", "layer.0.SelfAttention.k.weight": "k",
               "layer.0.SelfAttention.v.weight": "v", "layer.0.SelfAttention.o.weight": "o",
               "layer.0.SelfAttention.relative_attention_bias.weight": "rel_bias", "layer.0.layer_norm.weight": "ln0",
               "layer.1.DenseReluDense.wi_0.weight": "wi_0", "layer.1.DenseReluDense.wi_1.weight": "wi_1",
               "layer.1.DenseReluDense.wi.weight": "wi_0", "layer.1.DenseReluDense.wo.weight": "wo",
               "layer.1.layer_norm.weight": "ln1"}
        loaded = set()
        for name, w in weights:
            tgt = table.get(name)
            if tgt is None and name.startswith("encoder.block."):
                _, _, i, rest = name.split(".", 3)
                if rest in sub:
                    tgt = f"blocks.{i}.{sub[rest]}"
            if tgt is None or tgt not in params:
                continue
            params[tgt].data.copy_(w.to(params[tgt].dtype))
            loaded.add(tgt)
        return loaded


class T5EncoderModel(UMT5EncoderModel):
    per_layer_bias = False


def causal_position_bucket(rel: torch.Tensor, num_buckets: int, max_distance: int) -> torch.Tensor:
    """One-sided T5 bucketing of `key_pos - query_pos` for decoder self-attention (future keys fall in bucket 0)."""
    rel = (-rel).clamp_min(0)
    max_exact = num_buckets // 2
    small = rel < max_exact
    large = max_exact + (torch.log(rel.float().clamp_min(1) / max_exact) / math.log(max_distance / max_exact)
                         * (num_buckets - max_exact)).long()
    large = torch.minimum(large, torch.full_like(large, num_buckets - 1))
    return torch.where(small, rel, large)


class T5DecoderBlock(nn.Module):
    """Causal self-attention (with the relative-position bias), cross-attention over the encoder output, FFN."""

    def __init__(self, cfg, dtype, has_bias_table: bool):
        super().__init__()
        D, H, dk, F = cfg.d_model, cfg.num_heads, cfg.d_kv, cfg.d_ff
        self.H, self.dk = H, dk
        mk = lambda o, i: nn.Parameter(torch.empty(o, i, dtype=dtype), requires_grad=False)
        self.q, self.k, self.v, self.o = mk(H * dk, D), mk(H * dk, D), mk(H * dk, D), mk(D, H * dk)
        self.cq, self.ck, self.cv, self.co = mk(H * dk, D), mk(H * dk, D), mk(H * dk, D), mk(D, H * dk)
        self.rel_bias = nn.Parameter(torch.empty(cfg.relative_attention_num_buckets, H, dtype=dtype),
                                     requires_grad=False) if has_bias_table else None
        self.ln0, self.ln1, self.ln2 = (nn.Parameter(torch.ones(D, dtype=dtype), requires_grad=False) for _ in range(3))
        self.gated = bool(getattr(cfg, "is_gated_act", True))
        self.wi_0 = mk(F, D)
        self.wi_1 = mk(F, D) if self.gated else None
        self.wo = mk(D, F)
        act = getattr(cfg, "dense_act_fn", "gelu_new")
        self.act = (lambda t: torch.nn.functional.gelu(t, approximate="tanh")) if "gelu" in act else torch.relu
        self.eps = cfg.layer_norm_epsilon

    def _heads(self, h, w, B, T):
        return ops.linear(h.reshape(B * T, -1), w).view(B, T, self.H, self.dk).transpose(1, 2)

    def cross_kv(self, enc):
        """Keys / values of the encoder output `[B, S, D]`: computed once per prompt."""
        B, S, _ = enc.shape
        return self._heads(enc, self.ck, B, S), self._heads(enc, self.cv, B, S)

    def forward(self, x, bias, cross, enc_mask, cache=None):
        """`x [B, T, D]` (the new positions), `bias [1, H, T, past + T]` with the causal mask folded in, `cross` from
        `cross_kv`, `cache`: `(k, v)` of the earlier positions or None.  Returns `(x, (k, v))`."""
        B, T, D = x.shape
        h = _rms(x, self.ln0, self.eps)
        q, k, v = (self._heads(h, w, B, T) for w in (self.q, self.k, self.v))
        if cache is not None:
            k, v = torch.cat([cache[0], k], 2), torch.cat([cache[1], v], 2)
        s = torch.matmul(q.float(), k.float().transpose(-1, -2)) + bias
        a = torch.matmul(torch.softmax(s, -1), v.float()).to(x.dtype).transpose(1, 2).reshape(B * T, self.H * self.dk)
        x = x + ops.linear(a, self.o).view(B, T, D)
        h = _rms(x, self.ln1, self.eps)
        cq = self._heads(h, self.cq, B, T)
        s = torch.matmul(cq.float(), cross[0].float().transpose(-1, -2))
        if enc_mask is not None:
            s = s.masked_fill(~enc_mask[:, None, None, :], float("-inf"))
        a = torch.matmul(torch.softmax(s, -1), cross[1].float()).to(x.dtype).transpose(1, 2).reshape(B * T, -1)
        x = x + ops.linear(a, self.co).view(B, T, D)
        h = _rms(x, self.ln2, self.eps).reshape(B * T, D)
        g = self.act(ops.linear(h, self.wi_0))
        if self.gated:
            g = g * ops.linear(h, self.wi_1)
        return x + ops.linear(g, self.wo).view(B, T, D), (k, v)


class _T5DecoderStack(nn.Module):
    def __init__(self, config, dtype, per_layer_bias: bool):
        super().__init__()
        self.config = config
        n = getattr(config, "num_decoder_layers", None) or config.num_layers
        self.blocks = nn.ModuleList([T5DecoderBlock(config, dtype, per_layer_bias or i == 0) for i in range(n)])
        self.final_ln = nn.Parameter(torch.ones(config.d_model, dtype=dtype), requires_grad=False)

    def forward(self, x, enc, enc_mask, caches=None, cross=None):
        """`x [B, T, D]`: embeddings of the new decoder positions.  Returns `(hidden, caches, cross)`."""
        cfg = self.config
        T = x.shape[1]
        past = 0 if caches is None else caches[0][0].shape[2]
        qpos = torch.arange(past, past + T, device=x.device)
        kpos = torch.arange(past + T, device=x.device)
        rel = kpos[None, :] - qpos[:, None]
        buckets = causal_position_bucket(rel, cfg.relative_attention_num_buckets, cfg.relative_attention_max_distance)
        future = torch.zeros(rel.shape, device=x.device).masked_fill(rel > 0, float("-inf"))
        if cross is None:
            cross = [blk.cross_kv(enc) for blk in self.blocks]
        new_caches, bias = [], None
        for i, blk in enumerate(self.blocks):
            if blk.rel_bias is not None:
                bias = blk.rel_bias[buckets].permute(2, 0, 1).unsqueeze(0).float() + future
            x, kv = blk(x, bias, cross[i], enc_mask, None if caches is None else caches[i])
            new_caches.append(kv)
        return _rms(x, self.final_ln, cfg.layer_norm_epsilon), new_caches, cross


_DEC_SUB = {"layer.0.SelfAttention.q.weight": "q", "layer.0.SelfAttention.k.weight": "k",
            "layer.0.SelfAttention.v.weight": "v", "layer.0.SelfAttention.o.weight": "o",
            "layer.0.SelfAttention.relative_attention_bias.weight": "rel_bias", "layer.0.layer_norm.weight": "ln0",
            "layer.1.EncDecAttention.q.weight": "cq", "layer.1.EncDecAttention.k.weight": "ck",
            "layer.1.EncDecAttention.v.weight": "cv", "layer.1.EncDecAttention.o.weight": "co",
            "layer.1.layer_norm.weight": "ln1", "layer.2.DenseReluDense.wi_0.weight": "wi_0",
            "layer.2.DenseReluDense.wi_1.weight": "wi_1", "layer.2.DenseReluDense.wi.weight": "wi_0",
            "layer.2.DenseReluDense.wo.weight": "wo", "layer.2.layer_norm.weight": "ln2"}


def _load_decoder(params: dict, prefix: str, name: str, w: torch.Tensor) -> str | None:
    """Copy one `decoder.*` checkpoint tensor into the decoder stack registered under `prefix`."""
    tgt = None
    if name == "decoder.final_layer_norm.weight":
        tgt = f"{prefix}final_ln"
    elif name.startswith("decoder.block."):
        _, _, i, rest = name.split(".", 3)
        if rest in _DEC_SUB:
            tgt = f"{prefix}blocks.{i}.{_DEC_SUB[rest]}"
    if tgt is None or tgt not in params:
        return None
    params[tgt].data.copy_(w.to(params[tgt].dtype))
    return tgt


class UMT5DecoderModel(nn.Module):
    """The decoder stack alone: `forward(decoder_input_ids, encoder_hidden_states)`."""
    per_layer_bias = True

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        self.config = config
        self.shared = nn.Parameter(torch.empty(config.vocab_size, config.d_model, dtype=dtype), requires_grad=False)
        self.decoder = _T5DecoderStack(config, dtype, self.per_layer_bias)

    @torch.inference_mode()
    def forward(self, decoder_input_ids, encoder_hidden_states, encoder_attention_mask=None):
        mask = encoder_attention_mask.bool() if encoder_attention_mask is not None else None
        return self.decoder(self.shared[decoder_input_ids], encoder_hidden_states, mask)[0]

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            if name in ("shared.weight", "decoder.embed_tokens.weight"):
                params["shared"].data.copy_(w.to(params["shared"].dtype))
                loaded.add("shared")
            else:
                t = _load_decoder(params, "decoder.", name, w)
                if t:
                    loaded.add(t)
        return loaded


class UMT5Model(UMT5EncoderModel):
    """Encoder-decoder without a head: `forward(input_ids, decoder_input_ids)` -> decoder hidden states."""

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__(config, dtype, quant_config)
        self.decoder = _T5DecoderStack(config, dtype, self.per_layer_bias)

    @torch.inference_mode()
    def forward(self, input_ids, decoder_input_ids, attention_mask=None):
        enc = self.encode(input_ids, attention_mask)
        mask = attention_mask.bool() if attention_mask is not None else None
        return self.decoder(self.shared[decoder_input_ids], enc, mask)[0]

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        weights = list(weights)
        loaded = super().load_weights(weights)
        params = dict(self.named_parameters())
        for name, w in weights:
            t = _load_decoder(params, "decoder.", name, w)
            if t:
                loaded.add(t)
            elif name == "lm_head.weight" and "lm_head" in params:
                params["lm_head"].data.copy_(w.to(params["lm_head"].dtype))
                loaded.add("lm_head")
        return loaded


class UMT5ForConditionalGeneration(UMT5Model):
    """Encoder-decoder with the language-model head; `generate` is greedy with cached keys / values."""

    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__(config, dtype, quant_config)
        self.tied = bool(getattr(config, "tie_word_embeddings", False))
        if not self.tied:
            self.lm_head = nn.Parameter(torch.empty(config.vocab_size, config.d_model, dtype=dtype),
                                        requires_grad=False)

    def _logits(self, h):
        if self.tied:
            # tied checkpoints rescale before projecting onto the embedding table
            return ops.linear((h * self.config.d_model ** -0.5).reshape(-1, h.shape[-1]), self.shared).view(
                *h.shape[:-1], -1)
        return ops.linear(h.reshape(-1, h.shape[-1]), self.lm_head).view(*h.shape[:-1], -1)

    @torch.inference_mode()
    def forward(self, input_ids, decoder_input_ids, attention_mask=None):
        """Teacher-forced logits `[B, T_dec, vocab]`."""
        return self._logits(UMT5Model.forward(self, input_ids, decoder_input_ids, attention_mask))

    @torch.inference_mode()
    def generate(self, input_ids, max_new_tokens: int = 32, attention_mask=None, eos_token_id: int | None = None):
        """Greedy decoding from `decoder_start_token_id`; returns `[B, <= max_new_tokens]` new token ids (rows that
        finished early are padded with `pad_token_id`)."""
        cfg = self.config
        B = input_ids.shape[0]
        enc = self.encode(input_ids, attention_mask)
        mask = attention_mask.bool() if attention_mask is not None else None
        eos = getattr(cfg, "eos_token_id", None) if eos_token_id is None else eos_token_id
        pad = getattr(cfg, "pad_token_id", 0) or 0
        start = getattr(cfg, "decoder_start_token_id", None)
        cur = torch.full((B, 1), pad if start is None else start, dtype=torch.long, device=input_ids.device)
        caches = cross = None
        done = torch.zeros(B, dtype=torch.bool, device=input_ids.device)
        out = []
        for _ in range(max_new_tokens):
            h, caches, cross = self.decoder(self.shared[cur], enc, mask, caches, cross)
            nxt = self._logits(h[:, -1]).float().argmax(-1)
            nxt = torch.where(done, torch.full_like(nxt, pad), nxt)
            out.append(nxt)
            if eos is not None:
                done = done | (nxt == eos)
                if bool(done.all()):
                    break
            cur = nxt[:, None]
        return torch.stack(out, 1)


EntryClass = [UMT5EncoderModel, T5EncoderModel, UMT5DecoderModel, UMT5Model, UMT5ForConditionalGeneration]
