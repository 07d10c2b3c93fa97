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


class DefaultModelLoader:
    def __init__(self, load_format: str = "auto"):
        self.load_format = load_format

    def load_model(self, model_config, device, quant_config=None) -> torch.nn.Module:
        cls = get_model_class(model_config.architectures)
        with torch.device(device):
            model = cls(model_config.hf_config, dtype=model_config.dtype, quant_config=quant_config) \
                if _accepts_quant(cls) else cls(model_config.hf_config, dtype=model_config.dtype)
        it = self._iterator(model_config.model_path)
        loaded = model.load_weights(it)
        check_all_loaded(model, loaded)
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
        with torch.device(device):
            model = cls(model_config.hf_config, dtype=model_config.dtype, quant_config=quant_config) \
                if _accepts_quant(cls) else cls(model_config.hf_config, dtype=model_config.dtype)
        initialize_dummy_weights(model, self.seed)
        return model.eval()


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
