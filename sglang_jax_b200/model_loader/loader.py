"""Model construction and checkpoint loading.

Reference: `python/sgl_jax/srt/model_loader/loader.py` (`JAXModelLoader` :170, safetensors
iterator :149-167, `JAXDummyModelLoader` :325, `get_model_loader` :368) and
`python/sgl_jax/srt/utils/weight_utils.py` (`WeightLoader` :152).  Differences: the model is
built directly on its device under `torch.device(...)`, each rank reads only the slices it
owns (safetensors `get_slice` is lazy), and `dummy` fills seeded normal(0, 0.02) weights —
zeros (what the reference's dummy loader writes, `weight_utils.py:2360`) would make every
benchmark GEMM trivially compressible and every argmax a tie.
"""

from __future__ import annotations

import glob
import json
import logging
import os
from typing import Iterable

import torch

from ..models.registry import get_model_class

logger = logging.getLogger(__name__)


def safetensors_weights_iterator(model_path: str) -> Iterable[tuple[str, torch.Tensor]]:
    from safetensors import safe_open
    files = sorted(glob.glob(os.path.join(model_path, "*.safetensors")))
    idx = os.path.join(model_path, "model.safetensors.index.json")
    if os.path.isfile(idx):
        with open(idx) as f:
            wanted = set(json.load(f)["weight_map"].values())
        files = [f for f in files if os.path.basename(f) in wanted]
    if not files:
        raise FileNotFoundError(f"no *.safetensors under {model_path}")
    for fn in files:
        with safe_open(fn, framework="pt", device="cpu") as f:
            for name in f.keys():
                yield name, f.get_tensor(name)


def pt_weights_iterator(model_path: str):
    for fn in sorted(glob.glob(os.path.join(model_path, "*.bin")) + glob.glob(os.path.join(model_path, "*.pt"))):
        sd = torch.load(fn, map_location="cpu", weights_only=True)
        yield from sd.items()


def initialize_dummy_weights(model: torch.nn.Module, seed: int = 0, std: float = 0.02):
    """Seeded normal(0, std) for matrices, ones for norm scales, zeros for biases.  The
    generator is advanced per parameter *name* so every tensor-parallel rank draws the same
    full tensor statistics regardless of its shard."""
    for name, p in model.named_parameters():
        if p.dim() == 1:
            if "norm" in name or name.endswith("layernorm.weight"):
                p.data.fill_(1.0)
            else:
                p.data.zero_()
            continue
        g = torch.Generator(device=p.device)
        g.manual_seed((seed * 1_000_003 + hash_name(name)) % (2 ** 31))
        if p.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            tmp = torch.empty(p.shape, dtype=torch.bfloat16, device=p.device).normal_(0, 1.0, generator=g)
            p.data.copy_(tmp.to(p.dtype))
        else:
            p.data.normal_(0, std, generator=g)
    if hasattr(model, "post_load_weights"):
        model.post_load_weights()


def hash_name(name: str) -> int:
    h = 2166136261
    for ch in name.encode():
        h = ((h ^ ch) * 16777619) & 0xFFFFFFFF
    return h


def _expert_storage_for(quant_config):
    """Dynamic W8A8 e4m3 per-channel recipes build the routed experts directly in e4m3 storage, so a model whose
    bf16 experts would not fit on the device can still be loaded (each expert is quantised as it arrives)."""
    from ..layers.moe import expert_storage
    fp8 = torch.float8_e4m3fn
    if quant_config is None or quant_config.moe_weight_dtype != fp8:
        return expert_storage(None)
    block = tuple(quant_config.moe_weight_block_size or ()) or None
    if quant_config.is_static_checkpoint:
        # block-scaled fp8 release checkpoints (DeepSeek-V3): the experts stay e4m3 with their 128 x 128 scales
        return expert_storage(fp8 if block == (128, 128) else None, block)
    if quant_config.moe_activation_dtype != fp8 or (block and block != (128, 128)):
        return expert_storage(None)
    return expert_storage(fp8, block)


def _apply_dynamic_quantization(model, quant_config):
    """Dynamic recipes quantise the loaded (or dummy-initialised) bf16 weights in place.  Static 128 x 128
    block-scaled fp8 checkpoints take the same pass: their tensors arrive de-quantised from the iterator and are
    put back on the checkpoint's own block grid, so the dense projections end up in fp8 storage as well."""
    if quant_config is None:
        return
    if quant_config.is_static_checkpoint and tuple(getattr(quant_config, "weight_block_size", None) or ()) != (128, 128):
        return
    from ..utils.quantization import apply_linear_quantization, apply_moe_quantization
    n = apply_linear_quantization(model, quant_config) + apply_moe_quantization(model, quant_config)
    logger.info("quantized %d modules with recipe %s", n, quant_config.name)


class DefaultModelLoader:
    def __init__(self, load_format: str = "auto"):
        self.load_format = load_format

    def load_model(self, model_config, device, quant_config=None) -> torch.nn.Module:
        cls = get_model_class(model_config.architectures)
        with torch.device(device), _expert_storage_for(quant_config):
            model = cls(model_config.hf_config, dtype=model_config.dtype, quant_config=quant_config) \
                if _accepts_quant(cls) else cls(model_config.hf_config, dtype=model_config.dtype)
        it = self._iterator(model_config.model_path)
        pre = getattr(model, "preprocess_checkpoint", None)
        if pre is not None:
            # checkpoint tensors whose layout the generic passes below would misread (e.g. a fused projection that was
            # quantised shard by shard) are rewritten by the model first
            it = pre(it)
        it = dequant_static_fp8(it, getattr(quant_config, "weight_block_size", None))
        loaded = model.load_weights(it)
        check_all_loaded(model, loaded)
        _apply_dynamic_quantization(model, quant_config)
        _apply_dtype_config(model, model_config)
        return model.eval()

    def _iterator(self, path):
        if self.load_format in ("auto", "safetensors"):
            if glob.glob(os.path.join(path, "*.safetensors")):
                return safetensors_weights_iterator(path)
            if self.load_format == "safetensors":
                raise FileNotFoundError(f"no *.safetensors under {path}")
        if self.load_format in ("auto", "pt"):
            return pt_weights_iterator(path)
        raise NotImplementedError(f"load_format={self.load_format} is not implemented "
                                  f"(implemented: auto, safetensors, pt, dummy)")


class DummyModelLoader:
    def __init__(self, seed: int = 0):
        self.seed = seed

    def load_model(self, model_config, device, quant_config=None) -> torch.nn.Module:
        cls = get_model_class(model_config.architectures)
        with torch.device(device), _expert_storage_for(quant_config):
            model = cls(model_config.hf_config, dtype=model_config.dtype, quant_config=quant_config) \
                if _accepts_quant(cls) else cls(model_config.hf_config, dtype=model_config.dtype)
        initialize_dummy_weights(model, self.seed)
        _apply_dynamic_quantization(model, quant_config)
        _apply_dtype_config(model, model_config)
        return model.eval()


def _apply_dtype_config(model, model_config):
    """`--dtype-config`: per-module parameter dtypes (`configs/dtype_config.py`)."""
    cfg = getattr(model_config, "dtype_config", None)
    if cfg is None:
        return
    from ..configs.dtype_config import apply_dtype_config
    changed = apply_dtype_config(model, cfg)
    logger.info("dtype config changed %d parameters, e.g. %s", len(changed), list(changed.items())[:3])


def dequant_static_fp8(weights, block_size=None):
    """Static block-FP8 checkpoints (DeepSeek-V3 release format) ship `X.weight` in float8_e4m3fn
    next to `X.weight_scale_inv` ([ceil(N/128), ceil(K/128)] fp32).  The pair is multiplied out into one
    fp32 tensor while streaming, whatever order the two arrive in; everything else passes through.  The
    layers' loaders shard that tensor like any other weight, and for the 128 x 128 format the quantisation pass
    after loading puts it back on the checkpoint's own block grid in e4m3 storage (in a bf16 model the detour
    through the bf16 parameter leaves the e4m3 values unchanged and moves a block's scale by at most 2^-9)."""
    from ..utils.quantization import dequantize_tensor
    bs = tuple(block_size) if block_size else (128, 128)
    pend_w: dict[str, torch.Tensor] = {}
    pend_s: dict[str, torch.Tensor] = {}
    fp8 = (torch.float8_e4m3fn, torch.float8_e5m2)
    for name, w in weights:
        if name.endswith(".weight_scale_inv") or name.endswith(".weight_scale"):
            base = name.rsplit(".", 1)[0] + ".weight"
            inv = name.endswith("_inv")
            if base in pend_w:
                yield base, _fold(pend_w.pop(base), w, bs, inv, dequantize_tensor)
            else:
                pend_s[base] = (w, inv)
            continue
        if w.dtype in fp8:
            if name in pend_s:
                sc, inv = pend_s.pop(name)
                yield name, _fold(w, sc, bs, inv, dequantize_tensor)
            else:
                pend_w[name] = w
            continue
        yield name, w
    for name, w in pend_w.items():      # fp8 tensors without a scale: plain cast
        yield name, w.to(torch.float32)


def _fold(w, scale, bs, inv, dequantize_tensor):
    # both `weight_scale_inv` (DeepSeek) and `weight_scale` hold the multiplier that restores the weight
    if scale.dim() == 1 and scale.numel() == w.shape[0]:
        scale = scale.view(-1, 1)
    return dequantize_tensor(w, scale.float(), bs, torch.float32)


def check_all_loaded(model, loaded):
    """A parameter the checkpoint did not provide would silently stay uninitialised memory."""
    if loaded is None:
        return
    tied = {"lm_head.weight"} if getattr(model, "tie", False) else set()
    optional = getattr(model, "optional_params", set())
    missing = [n for n, _ in model.named_parameters() if n not in loaded and n not in tied
               and not any(n.endswith(o) for o in optional)]
    if missing:
        raise RuntimeError(f"checkpoint is missing {len(missing)} parameters, e.g. {missing[:5]}")


def _accepts_quant(cls) -> bool:
    import inspect
    return "quant_config" in inspect.signature(cls.__init__).parameters


def get_model_loader(load_format: str, seed: int = 0):
    if load_format == "dummy":
        return DummyModelLoader(seed)
    return DefaultModelLoader(load_format)
