"""Checkpoint ingestion shared by the sparse decoder families: name rewrites, stacked
q/k/v and gate/up projections, per-expert or fused expert tensors, router correction bias."""

from __future__ import annotations

import re
from typing import Iterable

import torch

STACKED = [
    (".qkv_proj", ".q_proj", "q"), (".qkv_proj", ".k_proj", "k"), (".qkv_proj", ".v_proj", "v"),
    (".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1),
]
_EXPERT_RE = re.compile(r"^(.*\.experts)\.(\d+)\.(\w+)\.weight$")


def load_sparse_weights(model, weights: Iterable[tuple[str, torch.Tensor]], renames: list[tuple[str, str]] = (),
                        expert_proj: dict | None = None, skip: tuple[str, ...] = (), max_layer: int | None = None,
                        stacked=STACKED) -> set:
    """`expert_proj` maps the checkpoint's per-expert projection names to `gate` / `up` / `down`
    (default HF `gate_proj`/`up_proj`/`down_proj`)."""
    expert_proj = expert_proj or {"gate_proj": "gate", "up_proj": "up", "down_proj": "down"}
    params = dict(model.named_parameters())
    modules = dict(model.named_modules())
    loaded: set = set()
    tie = bool(getattr(model, "tie", False))
    for name, w in weights:
        if "rotary_emb.inv_freq" in name or any(s in name for s in skip):
            continue
        for a, b in renames:
            name = name.replace(a, b)
        if max_layer is not None and name.startswith("model.layers."):
            if int(name.split(".")[2]) >= max_layer:
                continue
        if name == "lm_head.weight" and tie:
            continue
        m = _EXPERT_RE.match(name)
        if m and m.group(3) in expert_proj:
            head, e, shard = m.group(1), int(m.group(2)), expert_proj[m.group(3)]
            pname = f"{head}." + ("w2_weight" if shard == "down" else "w13_weight")
            if pname in params:
                p = params[pname]
                modules[head].weight_loader(p, w, shard, e)
                loaded.add(pname)
            continue
        if name.endswith(".experts.gate_up_proj") or name.endswith(".experts.down_proj"):
            head = name.rsplit(".", 1)[0]
            mod = modules[head]
            if name.endswith("gate_up_proj"):
                p = params[f"{head}.w13_weight"]
                half = w.shape[1] // 2
                for e in range(w.shape[0]):
                    mod.weight_loader(p, w[e, :half], "gate", e)
                    mod.weight_loader(p, w[e, half:], "up", e)
                loaded.add(f"{head}.w13_weight")
            else:
                p = params[f"{head}.w2_weight"]
                for e in range(w.shape[0]):
                    mod.weight_loader(p, w[e], "down", e)
                loaded.add(f"{head}.w2_weight")
            continue
        if name.endswith("e_score_correction_bias"):
            p = params.get(name)
            if p is not None:
                p.data.copy_(w.float())
                loaded.add(name)
            continue
        target, shard = name, None
        for pfrag, cfrag, sid in stacked:
            if cfrag in name:
                target, shard = name.replace(cfrag, pfrag), sid
                break
        if target not in params:
            continue
        mod = modules[target.rsplit(".", 1)[0]]
        p = params[target]
        mod.weight_loader(p, w.to(p.dtype) if w.dtype != p.dtype else w, shard)
        loaded.add(target)
    if hasattr(model, "post_load_weights"):
        model.post_load_weights()
    return loaded
