"""Loads adapters, owns the device pool, attaches the LoRA hooks to a model and prepares the
per-batch routing (reference `python/sgl_jax/srt/lora/lora_manager.py`)."""

from __future__ import annotations

import logging

import numpy as np
import torch

from ..layers.linear import (MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear)
from .backend.base_backend import LoRABatchInfo
from .backend.bgmv_backend import BgmvBackend
from .layers import LoRALinear, wrap_linear
from .lora import LoRAAdapter
from .lora_config import ALL_TARGETS, LoRAConfig, fused_targets
from .lora_memory_pool import LoRAMemoryPool
from .lora_registry import LoRARef, parse_lora_paths

logger = logging.getLogger(__name__)


class LoRAManager:
    def __init__(self, model: torch.nn.Module, server_args, dtype, device):
        self.model = model
        self.server_args = server_args
        self.dtype = dtype
        self.device = device
        self.adapters: dict[str, LoRAAdapter] = {}          # lora_id -> host weights
        self.refs: dict[str, LoRARef] = {}
        self.max_loaded = server_args.max_loaded_loras
        refs = parse_lora_paths(server_args.lora_paths)
        configs = [LoRAConfig(r.lora_path) for r in refs]
        self.max_rank = int(server_args.max_lora_rank or max([c.r for c in configs], default=0))
        if self.max_rank <= 0:
            raise ValueError("LoRA needs --max-lora-rank or at least one adapter in --lora-paths")
        targets = server_args.lora_target_modules or sorted({m for c in configs for m in c.target_modules}) or ALL_TARGETS
        self.target_modules = fused_targets(list(targets))
        self.backend = BgmvBackend()
        self.pool = LoRAMemoryPool(server_args.max_loras_per_batch, self.max_rank, dtype, device,
                                   server_args.lora_eviction_policy)
        self._attach()
        for ref in refs:
            res = self.load_adapter(ref)
            if not res[0]:
                raise ValueError(res[1])
        logger.info("LoRA: %d adapters, rank<=%d, targets=%s, pool %.1f MB", len(self.adapters), self.max_rank,
                    self.target_modules, self.pool.get_buffer_bytes() / 2 ** 20)

    # ------------------------------------------------------------------ model surgery
    def _attach(self):
        import re
        pat = re.compile(r"layers\.(\d+)\.(?:.*\.)?(qkv_proj|gate_up_proj|o_proj|down_proj)$")
        n = 0
        for name, mod in self.model.named_modules():
            m = pat.search(name)
            if m is None or m.group(2) not in self.target_modules:
                continue
            layer, kind = int(m.group(1)), m.group(2)
            shard = self._shard_of(mod)
            if shard is None:
                continue
            a, bs = self.pool.add_module(layer, kind, mod, shard)
            offs = list(np.cumsum([0] + [l for _, l in shard["out_slices"]])[:-1])
            wrap_linear(mod, LoRALinear(kind, layer, self.backend, a, bs, [int(o) for o in offs]))
            n += 1
        if n == 0:
            raise ValueError(f"no module of the model matches LoRA targets {self.target_modules}")

    @staticmethod
    def _shard_of(mod) -> dict | None:
        if isinstance(mod, QKVParallelLinear):
            hd = mod.head_dim
            q_tot = mod.total_num_heads * hd
            k_tot = mod.total_num_kv_heads * hd
            kv_idx = mod.tp_rank // mod.num_kv_head_replicas
            return dict(kind="column", in_slice=(0, mod.in_features),
                        out_slices=[(mod.tp_rank * mod.q_size, mod.q_size), (kv_idx * mod.k_size, mod.k_size),
                                    (kv_idx * mod.v_size, mod.v_size)],
                        fused_out_starts=[mod.tp_rank * mod.q_size, q_tot + kv_idx * mod.k_size,
                                          q_tot + k_tot + kv_idx * mod.v_size])
        if isinstance(mod, MergedColumnParallelLinear):
            starts, acc = [], 0
            for full, loc in zip(mod.output_sizes, mod.local_sizes):
                starts.append(acc + mod.tp_rank * loc)
                acc += full
            return dict(kind="column", in_slice=(0, mod.in_features),
                        out_slices=[(mod.tp_rank * loc, loc) for loc in mod.local_sizes], fused_out_starts=starts)
        if isinstance(mod, RowParallelLinear):
            return dict(kind="row", in_slice=(mod.tp_rank * mod.in_features, mod.in_features),
                        out_slices=[(0, mod.out_features)], fused_out_starts=[0])
        return None

    # ------------------------------------------------------------------ adapters
    def load_adapter(self, ref: LoRARef) -> tuple[bool, str]:
        if ref.lora_id in self.adapters:
            return False, f"LoRA adapter {ref.lora_name} is already loaded"
        if self.max_loaded is not None and len(self.adapters) >= self.max_loaded:
            return False, f"cannot load {ref.lora_name}: --max-loaded-loras={self.max_loaded} reached"
        try:
            ad = LoRAAdapter.from_path(ref.lora_id, ref.lora_path)
        except Exception as e:  # noqa: BLE001
            return False, f"failed to load LoRA adapter {ref.lora_name} from {ref.lora_path}: {e}"
        if ad.r > self.max_rank:
            return False, f"LoRA adapter {ref.lora_name} has rank {ad.r} > max_lora_rank {self.max_rank}"
        extra = set(fused_targets(ad.config.target_modules)) - set(self.target_modules)
        if extra:
            return False, (f"LoRA adapter {ref.lora_name} targets {sorted(extra)}, which --lora-target-modules "
                           f"does not cover")
        if self.server_args.lora_scaling is not None:
            ad.scaling = float(self.server_args.lora_scaling)
        self.adapters[ref.lora_id] = ad
        self.refs[ref.lora_id] = ref
        return True, ""

    def unload_adapter(self, lora_id: str) -> tuple[bool, str]:
        if lora_id not in self.adapters:
            return False, f"LoRA adapter id {lora_id} is not loaded"
        del self.adapters[lora_id]
        self.refs.pop(lora_id, None)
        self.pool.evict(lora_id)
        return True, ""

    def loaded(self) -> dict[str, str]:
        return {r.lora_name: r.lora_path for r in self.refs.values()}

    # ------------------------------------------------------------------ per batch
    def prepare_batch(self, lora_ids: list | None, tokens_per_req: np.ndarray) -> LoRABatchInfo | None:
        """`lora_ids[b]` is the adapter of request b (None = base model); `tokens_per_req[b]` its
        number of rows in this forward."""
        if not lora_ids or all(i is None for i in lora_ids):
            return None
        uids = {i for i in lora_ids if i is not None}
        missing = uids - set(self.adapters)
        if missing:
            raise ValueError(f"LoRA adapter ids {sorted(missing)} are not loaded")
        slots = self.pool.prepare(uids, self.adapters)
        per_req = np.asarray([slots[i] if i is not None else -1 for i in lora_ids], np.int32)
        tok = np.repeat(per_req, np.asarray(tokens_per_req, np.int64))
        order = np.argsort(tok, kind="stable")
        sorted_slots = tok[order]
        start = int(np.searchsorted(sorted_slots, 0))
        seg_slots, seg_bounds = [], []
        i = start
        while i < len(order):
            j = int(np.searchsorted(sorted_slots, sorted_slots[i], side="right"))
            seg_slots.append(int(sorted_slots[i]))
            seg_bounds.append((i - start, j - start))
            i = j
        return LoRABatchInfo(
            token_slots=torch.from_numpy(tok).to(self.device), scalings=self.pool.scalings, ranks=self.pool.ranks,
            has_lora=True, order=torch.from_numpy(order[start:].astype(np.int64)).to(self.device),
            seg_slots=seg_slots, seg_bounds=seg_bounds)
