"""Token embedding, LM head and rotary position embeddings.

Reference: `python/sgl_jax/srt/layers/embeddings.py` (`Embed` :32, `ParallelLMHead` :127,
`RotaryEmbedding` :192, `MRotaryEmbedding` :308, `ProportionalRotaryEmbedding` :455,
`Llama3RotaryEmbedding` :494, `YarnRotaryEmbedding` :763, `get_rope` :604).
Each rotary variant only differs in how it builds the fp32 `[max_pos, rotary_dim]`
cos|sin table; applying it is one fused kernel shared with the q/k norm and the KV write
(`ops.rope_qknorm_kvwrite`).
"""

from __future__ import annotations

import math

import torch
from torch import nn

from .. import ops
from ..ops import reference
from ..parallel import state as ps


def pad_vocab(vocab_size: int, tp: int, multiple: int = 64) -> int:
    m = multiple * tp
    return (vocab_size + m - 1) // m * m


class VocabParallelEmbedding(nn.Module):
    """Embedding table.  On B200 the table is replicated on every tensor rank (1.5 GB for a
    152k x 5120 bf16 table is noise next to 180 GB of HBM) which removes the all-reduce the
    vocab-sharded layout of the reference needs (`embeddings.py:32-125`).  `shard=True`
    restores the sharded layout + all-reduce for memory-tight deployments."""

    def __init__(self, num_embeddings, embedding_dim, dtype=torch.bfloat16, shard: bool = False,
                 tp_size=None, tp_rank=None):
        super().__init__()
        self.tp_size = (tp_size if tp_size is not None else ps.tp_size()) if shard else 1
        self.tp_rank = (tp_rank if tp_rank is not None else ps.tp_rank()) if shard else 0
        self.num_embeddings = num_embeddings
        self.padded = pad_vocab(num_embeddings, self.tp_size)
        self.local = self.padded // self.tp_size
        self.vocab_start = self.tp_rank * self.local
        self.weight = nn.Parameter(torch.zeros(self.local, embedding_dim, dtype=dtype), requires_grad=False)
        self.out_dtype = dtype            # the activations' dtype, also when `--dtype-config` stores the table wider

    def weight_loader(self, param, w, shard_id=None):
        lo = self.vocab_start
        hi = min(lo + self.local, w.shape[0])
        if hi > lo:
            param.data[: hi - lo].copy_(w[lo:hi])

    def forward(self, ids):
        if self.tp_size == 1:
            out = ops.embedding(ids, self.weight)
            return out if out.dtype == self.out_dtype else out.to(self.out_dtype)
        out = ops.embedding(ids, self.weight, self.vocab_start, masked=True)
        out = ps.all_reduce(out)
        return out if out.dtype == self.out_dtype else out.to(self.out_dtype)


class ParallelLMHead(nn.Module):
    """Vocab-parallel output projection; each rank holds `[vocab/tp, hidden]`."""

    def __init__(self, num_embeddings, embedding_dim, dtype=torch.bfloat16, tp_size=None, tp_rank=None):
        super().__init__()
        self.tp_size = tp_size if tp_size is not None else ps.tp_size()
        self.tp_rank = tp_rank if tp_rank is not None else ps.tp_rank()
        self.num_embeddings = num_embeddings
        self.padded = pad_vocab(num_embeddings, self.tp_size)
        self.local = self.padded // self.tp_size
        self.vocab_start = self.tp_rank * self.local
        self.weight = nn.Parameter(torch.zeros(self.local, embedding_dim, dtype=dtype), requires_grad=False)

    def weight_loader(self, param, w, shard_id=None):
        lo = self.vocab_start
        hi = min(lo + self.local, w.shape[0])
        if hi > lo:
            param.data[: hi - lo].copy_(w[lo:hi])

    def tie_to(self, embed: VocabParallelEmbedding):
        w = embed.weight
        if w.shape[0] == self.local and self.tp_size == 1:
            self.weight = w
        else:
            lo = self.vocab_start
            hi = min(lo + self.local, w.shape[0])
            self.weight.data.zero_()
            self.weight.data[: hi - lo].copy_(w.data[lo:hi])


# ------------------------------------------------------------------------------ rotary
class RotaryEmbedding(nn.Module):
    def __init__(self, head_size, rotary_dim, max_position_embeddings, base, is_neox_style=True,
                 dtype=torch.bfloat16):
        super().__init__()
        self.head_size = head_size
        self.rotary_dim = rotary_dim
        self.max_position_embeddings = max_position_embeddings
        self.base = base
        self.is_neox_style = is_neox_style
        self.register_buffer("cos_sin_cache", self._compute_cos_sin_cache(), persistent=False)

    def _compute_inv_freq(self, base) -> torch.Tensor:
        return 1.0 / (base ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float32, device="cpu") / self.rotary_dim))

    def _mscale(self) -> float:
        return 1.0

    def _compute_cos_sin_cache(self) -> torch.Tensor:
        return reference.build_cos_sin_cache(self.rotary_dim, self.max_position_embeddings, self.base,
                                             self._compute_inv_freq(self.base), self._mscale())

    def forward(self, positions, q, k):
        """Standalone application on `[T, H, D]` tensors (models normally use the fused op)."""
        return (reference.apply_rope(q, positions, self.cos_sin_cache, self.is_neox_style, self.rotary_dim),
                reference.apply_rope(k, positions, self.cos_sin_cache, self.is_neox_style, self.rotary_dim))


class Llama3RotaryEmbedding(RotaryEmbedding):
    def __init__(self, head_size, rotary_dim, max_pos, base, is_neox_style, dtype, scaling_factor,
                 low_freq_factor, high_freq_factor, orig_max_position):
        self.scaling_factor = scaling_factor
        self.low_freq_factor = low_freq_factor
        self.high_freq_factor = high_freq_factor
        self.orig_max_position = orig_max_position
        super().__init__(head_size, rotary_dim, max_pos, base, is_neox_style, dtype)

    def _compute_inv_freq(self, base):
        inv = super()._compute_inv_freq(base)
        low_wl = self.orig_max_position / self.low_freq_factor
        high_wl = self.orig_max_position / self.high_freq_factor
        wl = 2 * math.pi / inv
        smooth = (self.orig_max_position / wl - self.low_freq_factor) / (self.high_freq_factor - self.low_freq_factor)
        scaled = torch.where(wl < high_wl, inv,
                             torch.where(wl > low_wl, inv / self.scaling_factor,
                                         (1 - smooth) * inv / self.scaling_factor + smooth * inv))
        return scaled


def _yarn_find_correction_dim(num_rot, dim, base, max_pos):
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def yarn_get_mscale(scale: float = 1.0, mscale: float = 1.0) -> float:
    if scale <= 1:
        return 1.0
    return 0.1 * mscale * math.log(scale) + 1.0


class YarnRotaryEmbedding(RotaryEmbedding):
    """YaRN / DeepSeek-YaRN scaling."""

    def __init__(self, head_size, rotary_dim, orig_max_pos, base, is_neox_style, dtype, scaling_factor,
                 extrapolation_factor=1.0, attn_factor=1.0, beta_fast=32, beta_slow=1, mscale=1.0,
                 mscale_all_dim=0.0, deepseek: bool = False):
        self.scaling_factor = scaling_factor
        self.extrapolation_factor = extrapolation_factor
        self.attn_factor = attn_factor
        self.beta_fast, self.beta_slow = beta_fast, beta_slow
        self.orig_max_pos = orig_max_pos
        if deepseek:
            self.mscale_value = yarn_get_mscale(scaling_factor, mscale) / yarn_get_mscale(scaling_factor, mscale_all_dim) * attn_factor
        else:
            self.mscale_value = yarn_get_mscale(scaling_factor) * attn_factor
        super().__init__(head_size, rotary_dim, int(orig_max_pos * scaling_factor), base, is_neox_style, dtype)

    def _mscale(self):
        return self.mscale_value

    def _compute_inv_freq(self, base):
        pos_freqs = base ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float32, device="cpu") / self.rotary_dim)
        extra = 1.0 / pos_freqs
        inter = 1.0 / (self.scaling_factor * pos_freqs)
        low = max(math.floor(_yarn_find_correction_dim(self.beta_fast, self.rotary_dim, base, self.orig_max_pos)), 0)
        high = min(math.ceil(_yarn_find_correction_dim(self.beta_slow, self.rotary_dim, base, self.orig_max_pos)),
                   self.rotary_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(self.rotary_dim // 2, dtype=torch.float32, device="cpu") - low) / (high - low)).clamp(0, 1)
        mask = (1 - ramp) * self.extrapolation_factor
        return inter * (1 - mask) + extra * mask


class ProportionalRotaryEmbedding(RotaryEmbedding):
    """Rotates only the first `partial_rotary_factor` of the frequency spectrum and leaves the
    rest of the head un-rotated by giving those lanes zero frequency (Gemma-4 global layers)."""

    def __init__(self, head_size, rotary_dim, max_pos, base, is_neox_style, dtype, partial_rotary_factor=1.0):
        self.partial = partial_rotary_factor
        super().__init__(head_size, rotary_dim, max_pos, base, is_neox_style, dtype)

    def _compute_inv_freq(self, base):
        half = self.rotary_dim // 2
        n_rot = int(half * self.partial)
        inv = 1.0 / (base ** (torch.arange(0, 2 * n_rot, 2, dtype=torch.float32, device="cpu") / self.rotary_dim))
        return torch.cat([inv, torch.zeros(half - n_rot, device="cpu")])


class MRotaryEmbedding(RotaryEmbedding):
    """Multimodal RoPE (Qwen2-VL family): positions are `[3, T]` (temporal, height, width) and
    the frequency lanes are partitioned into `mrope_section` groups, each driven by one of the
    three position streams."""

    def __init__(self, head_size, rotary_dim, max_pos, base, is_neox_style, dtype, mrope_section,
                 interleaved: bool = False):
        self.mrope_section = mrope_section
        # interleaved layout (Qwen3-VL / Qwen3-Omni): lanes cycle T, H, W, T, H, W, ... while a
        # stream still has lanes left in its section; the remainder follows the temporal stream
        self.mrope_interleaved = interleaved
        super().__init__(head_size, rotary_dim, max_pos, base, is_neox_style, dtype)

    def forward(self, positions, q, k):
        if positions.dim() == 1:
            return super().forward(positions, q, k)
        cs = self.cos_sin_cache[positions.long()]            # [3, T, rd]
        half = self.rotary_dim // 2
        cos, sin = cs[..., :half], cs[..., half:]
        if self.mrope_interleaved:
            cos, sin = cos[0].clone(), sin[0].clone()
            for i, off in ((1, 1), (2, 2)):
                sl = slice(off, self.mrope_section[i] * 3, 3)
                cos[:, sl], sin[:, sl] = cs[i, :, :half][:, sl], cs[i, :, half:][:, sl]
            cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
        else:
            parts_c, parts_s, o = [], [], 0
            for i, n in enumerate(self.mrope_section):
                parts_c.append(cos[i, :, o:o + n])
                parts_s.append(sin[i, :, o:o + n])
                o += n
            cos, sin = torch.cat(parts_c, -1).unsqueeze(1), torch.cat(parts_s, -1).unsqueeze(1)

        def rot(x):
            xf = x[..., : self.rotary_dim].float()
            x1, x2 = xf[..., :half], xf[..., half:]
            out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)
            if self.rotary_dim < x.shape[-1]:
                out = torch.cat([out, x[..., self.rotary_dim:].float()], -1)
            return out.to(x.dtype)

        return rot(q), rot(k)


_ROPE_CACHE: dict = {}


def get_rope(head_size, rotary_dim, max_position, base, is_neox_style=True, rope_scaling: dict | None = None,
             dtype=torch.bfloat16, partial_rotary_factor: float = 1.0) -> RotaryEmbedding:
    if partial_rotary_factor < 1.0 and not (rope_scaling or {}).get("proportional"):
        rotary_dim = int(rotary_dim * partial_rotary_factor)
    key = (head_size, rotary_dim, max_position, base, is_neox_style,
           tuple(sorted((k, str(v)) for k, v in (rope_scaling or {}).items())), partial_rotary_factor)
    if key in _ROPE_CACHE:
        return _ROPE_CACHE[key]
    rs = rope_scaling or {}
    kind = rs.get("rope_type", rs.get("type"))
    if kind in (None, "default", "linear"):
        if rs.get("proportional"):
            rope = ProportionalRotaryEmbedding(head_size, rotary_dim, max_position, base, is_neox_style, dtype,
                                               partial_rotary_factor)
        elif "mrope_section" in rs:
            rope = MRotaryEmbedding(head_size, rotary_dim, max_position, base, is_neox_style, dtype, rs["mrope_section"],
                                    bool(rs.get("mrope_interleaved", False)))
        else:
            rope = RotaryEmbedding(head_size, rotary_dim, max_position, base, is_neox_style, dtype)
    elif kind == "llama3":
        rope = Llama3RotaryEmbedding(head_size, rotary_dim, max_position, base, is_neox_style, dtype,
                                     rs["factor"], rs["low_freq_factor"], rs["high_freq_factor"],
                                     rs["original_max_position_embeddings"])
    elif kind in ("yarn", "deepseek_yarn"):
        extra = {k: rs[k] for k in ("extrapolation_factor", "attn_factor", "beta_fast", "beta_slow",
                                    "mscale", "mscale_all_dim") if k in rs}
        rope = YarnRotaryEmbedding(head_size, rotary_dim, rs.get("original_max_position_embeddings", max_position),
                                   base, is_neox_style, dtype, rs["factor"], deepseek=(kind == "deepseek_yarn"), **extra)
    elif kind == "mrope":
        rope = MRotaryEmbedding(head_size, rotary_dim, max_position, base, is_neox_style, dtype, rs["mrope_section"])
    else:
        raise ValueError(f"Unknown RoPE scaling type {kind}")
    _ROPE_CACHE[key] = rope
    return rope
