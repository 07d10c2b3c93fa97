"""Tensor quantisation helpers and the model-surgery pass that applies a recipe (reference
`python/sgl_jax/srt/utils/quantization/quantization_utils.py`: `apply_linear_quantization` :78,
`apply_moe_quantization` :224, `quantize_tensor` :317, `dequantize_tensor` :425)."""

from __future__ import annotations

import logging
import math

import torch
from torch import nn

from ..configs.quantization_config import QuantizationConfig

logger = logging.getLogger(__name__)

_QMAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0, torch.int8: 127.0}


def _cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    q = _QMAX[dtype]
    x = x.clamp(-q, q)
    return x.round().to(torch.int8) if dtype == torch.int8 else x.to(dtype)


def quantize_tensor(w: torch.Tensor, dtype: torch.dtype, granularity: str = "per_channel",
                    block_size: tuple[int, int] | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """`w [N, K]` -> `(q, scale)` with `w ~= q * scale` (scale broadcast per granularity):
    per_tensor `[]`, per_channel `[N, 1]`, block `[ceil(N/bn), ceil(K/bk)]`."""
    wf = w.float()
    qmax = _QMAX[dtype]
    if granularity == "per_tensor":
        scale = (wf.abs().max() / qmax).clamp_min(1e-12)
        return _cast(wf / scale, dtype), scale
    if granularity == "per_channel":
        scale = (wf.abs().amax(dim=-1, keepdim=True) / qmax).clamp_min(1e-12)
        return _cast(wf / scale, dtype), scale
    bn, bk = block_size or (128, 128)
    N, K = wf.shape
    nb, kb = math.ceil(N / bn), math.ceil(K / bk)
    pad = torch.zeros(nb * bn, kb * bk, dtype=torch.float32, device=w.device)
    pad[:N, :K] = wf
    blocks = pad.view(nb, bn, kb, bk)
    scale = (blocks.abs().amax(dim=(1, 3)) / qmax).clamp_min(1e-12)            # [nb, kb]
    q = (blocks / scale[:, None, :, None]).reshape(nb * bn, kb * bk)[:N, :K]
    return _cast(q, dtype), scale


def dequantize_tensor(q: torch.Tensor, scale: torch.Tensor, block_size: tuple[int, int] | None = None,
                      out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    qf = q.float()
    if scale.dim() == 0 or scale.numel() == 1:
        return (qf * scale.float()).to(out_dtype)
    if scale.dim() == 2 and scale.shape[-1] == 1 and scale.shape[0] == q.shape[0]:
        return (qf * scale.float()).to(out_dtype)
    bn, bk = block_size or (128, 128)
    N, K = q.shape
    s = scale.float().repeat_interleave(bn, 0)[:N].repeat_interleave(bk, 1)[:, :K]
    return (qf * s).to(out_dtype)


def quantize_activation(x: torch.Tensor, dtype: torch.dtype, group: int | None = None):
    """Per-token (`group=None`) or per-token-group (1 x `group`) dynamic activation scales."""
    xf = x.float()
    qmax = _QMAX[dtype]
    if group is None:
        s = (xf.abs().amax(-1, keepdim=True) / qmax).clamp_min(1e-12)
        return _cast(xf / s, dtype), s
    T, K = xf.shape
    kb = math.ceil(K / group)
    pad = torch.zeros(T, kb * group, dtype=torch.float32, device=x.device)
    pad[:, :K] = xf
    g = pad.view(T, kb, group)
    s = (g.abs().amax(-1) / qmax).clamp_min(1e-12)                              # [T, kb]
    return _cast((g / s[..., None]).reshape(T, kb * group)[:, :K], dtype), s


class QuantizedWeight(nn.Module):
    """Storage of one quantised `[N, K]` weight: `qweight` + `scale` (+ block size)."""

    def __init__(self, qweight: torch.Tensor, scale: torch.Tensor, block_size=None, act_dtype=None,
                 out_dtype=torch.bfloat16):
        super().__init__()
        self.qweight = nn.Parameter(qweight, requires_grad=False)
        self.scale = nn.Parameter(scale.float(), requires_grad=False)
        self.block_size = tuple(block_size) if block_size else None
        self.act_dtype = act_dtype
        self.out_dtype = out_dtype

    def dequantized(self) -> torch.Tensor:
        return dequantize_tensor(self.qweight, self.scale, self.block_size, self.out_dtype)

    def linear(self, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        """`x @ W^T` with the activation rounded through the recipe's activation dtype, fp32 accumulate."""
        from .. import ops
        if (self.act_dtype == torch.float8_e4m3fn and self.qweight.dtype == torch.float8_e4m3fn and self.block_size is None
                and self.scale.numel() == self.qweight.shape[0] and x.is_cuda and self.out_dtype == torch.bfloat16
                and not ops._FORCE_REFERENCE):
            # W8A8 e4m3 with per-channel weight scales and per-token activation scales: fp8 tensor-core GEMM
            native = ops._native()
            if native.gemm_fp8_supported(self.qweight, self.qweight) and x.shape[-1] % 16 == 0:
                x2 = x.reshape(-1, x.shape[-1])
                if x2.dtype == torch.bfloat16 and x2.shape[-1] % 8 == 0:
                    xq, xs = native.quant_fp8_rows(x2)
                else:
                    xq, xs = quantize_activation(x2, self.act_dtype, None)
                y = native.gemm_fp8(xq, self.qweight, xs, self.scale, bias)
                return y.view(*x.shape[:-1], self.qweight.shape[0])
        if (self.qweight.dtype == torch.float8_e4m3fn and self.block_size is not None and x.is_cuda
                and self.act_dtype in (torch.float8_e4m3fn, None) and self.out_dtype == torch.bfloat16
                and x.dtype == torch.bfloat16 and not ops._FORCE_REFERENCE):
            # 128 x 128 block-scaled weights (DeepSeek-V3 format) with per-token-group-128 activation scales:
            # the fp8 weights stay fp8 and every K block is promoted with its scales inside the GEMM
            native = ops._native()
            if native.gemm_fp8_block_supported(self.qweight, self.scale, self.block_size):
                x2 = x.reshape(-1, x.shape[-1])
                xq, xs = native.quant_fp8_group128(x2)
                y = native.gemm_fp8_block(xq, xs, self.qweight, self.scale, bias)
                return y.view(*x.shape[:-1], self.qweight.shape[0])
        if self.act_dtype is not None and self.act_dtype in _QMAX:
            xq, xs = quantize_activation(x.reshape(-1, x.shape[-1]), self.act_dtype,
                                         self.block_size[1] if self.block_size else None)
            if xs.dim() == 2 and xs.shape[1] > 1:
                xs = xs.repeat_interleave(self.block_size[1], 1)[:, : x.shape[-1]]
            x = (xq.float() * xs).to(self.out_dtype).view(x.shape)
        return ops.linear(x, self.dequantized(), bias)


def apply_linear_quantization(model: nn.Module, cfg: QuantizationConfig) -> int:
    """Quantise (dynamic recipes) every `LinearBase` the rules select, in place: the bf16 weight is
    replaced by `QuantizedWeight` storage and the layer's forward goes through it.  Returns how
    many layers changed."""
    from ..layers.linear import LinearBase
    n = 0
    for name, mod in model.named_modules():
        if not isinstance(mod, LinearBase) or getattr(mod, "qweight", None) is not None:
            continue
        if name.endswith("lm_head") or "embed" in name:
            continue        # vocabulary tables stay in the compute dtype
        rule = cfg.rule_for(name)
        if rule is None or mod.weight is None or mod.weight.dtype in _QMAX:
            continue
        gran = "block" if cfg.weight_block_size else cfg.granularity
        q, s = quantize_tensor(mod.weight.data, rule.weight_dtype, gran, cfg.weight_block_size)
        mod.set_quantized(QuantizedWeight(q, s, cfg.weight_block_size if gran == "block" else None,
                                          rule.activation_dtype, mod.weight.dtype))
        n += 1
    return n


def apply_moe_quantization(model: nn.Module, cfg: QuantizationConfig) -> int:
    from ..layers.moe import FusedMoE
    if cfg.moe_weight_dtype is None:
        return 0
    n = 0
    for _, mod in model.named_modules():
        if isinstance(mod, FusedMoE) and not getattr(mod, "quantized", False):
            mod.quantize_(cfg.moe_weight_dtype, cfg.moe_weight_block_size, cfg.moe_activation_dtype)
            n += 1
    return n


def attach_static_scales(model: nn.Module, scales: dict[str, torch.Tensor], cfg: QuantizationConfig) -> int:
    """Static checkpoints: `scales` maps `<module>.weight_scale_inv` to the block scales that came
    with the fp8 weights (which were loaded into the layers' weight tensors as raw fp8)."""
    from ..layers.linear import LinearBase
    mods = dict(model.named_modules())
    n = 0
    for key, s in scales.items():
        name = key.rsplit(".", 1)[0]
        mod = mods.get(name)
        if isinstance(mod, LinearBase) and mod.weight.dtype in _QMAX:
            mod.set_quantized(QuantizedWeight(mod.weight.data, s, cfg.weight_block_size, None, torch.bfloat16))
            n += 1
    return n
