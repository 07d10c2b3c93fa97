"""Command-line helpers around recorded expert loads (reference `scripts/analyze_hot_experts.py`,
`scripts/inspect_expert_dist.py`, `scripts/plot_expert_balance.py`).

    python -m sglang_jax_b200.eplb.tools inspect  counts.npy --topk 8
    python -m sglang_jax_b200.eplb.tools hot      counts.npy --num-devices 8
    python -m sglang_jax_b200.eplb.tools rebalance counts.npy --num-devices 8 --redundant 8

`counts.npy` is a `[layers, experts]` (or `[segments, layers, experts]`) array of routed-token
counts, e.g. the dump of `RoutedExpertsCapturer`."""

from __future__ import annotations

import argparse
import sys

import numpy as np


def load_counts(path: str) -> np.ndarray:
    d = np.load(path, allow_pickle=True)
    if d.dtype == object:
        d = d.item()
        key = next(k for k, v in d.items() if hasattr(v, "ndim") and v.ndim >= 2)
        d = np.asarray(d[key])
    return np.asarray(d, dtype=np.float64)


def hot_experts(counts: np.ndarray, topk: int = 8) -> list[list[tuple[int, float]]]:
    """Per layer: the `topk` experts by load with their ratio to the layer mean."""
    c = counts.reshape(-1, *counts.shape[-2:]).sum(0)
    out = []
    for row in c:
        mean = max(row.mean(), 1e-9)
        idx = np.argsort(-row)[:topk]
        out.append([(int(i), float(row[i] / mean)) for i in idx])
    return out


def device_imbalance(counts: np.ndarray, num_devices: int) -> np.ndarray:
    """`[layers]` max-over-mean device load with experts laid out contiguously."""
    c = counts.reshape(-1, *counts.shape[-2:]).sum(0)
    L, E = c.shape
    per = c.reshape(L, num_devices, E // num_devices).sum(-1)
    return per.max(-1) / np.maximum(per.mean(-1), 1e-9)


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("inspect", "hot", "rebalance"):
        p = sub.add_parser(name)
        p.add_argument("path")
        p.add_argument("--topk", type=int, default=8)
        p.add_argument("--num-devices", type=int, default=8)
        p.add_argument("--redundant", type=int, default=0)
        p.add_argument("--csv", default=None)
    a = ap.parse_args(argv)
    counts = load_counts(a.path)
    if a.cmd == "inspect":
        print(f"shape={counts.shape} total={counts.sum():.0f}")
        for layer, pairs in enumerate(hot_experts(counts, a.topk)):
            print(f"layer {layer:3d}: " + " ".join(f"e{e}x{r:.2f}" for e, r in pairs))
    elif a.cmd == "hot":
        imb = device_imbalance(counts, a.num_devices)
        for layer, v in enumerate(imb):
            print(f"layer {layer:3d}: device max/mean = {v:.3f}")
        print(f"worst layer {int(imb.argmax())}: {imb.max():.3f}; mean {imb.mean():.3f}")
    else:
        from .expert_location import rebalance
        c = counts.reshape(-1, *counts.shape[-2:]).sum(0)
        num_phy = c.shape[1] + a.redundant
        phy2log = np.stack([rebalance(c[layer], num_phy, a.num_devices) for layer in range(c.shape[0])])
        before = device_imbalance(counts, a.num_devices)
        after = []
        for layer in range(c.shape[0]):
            reps = np.bincount(phy2log[layer], minlength=c.shape[1]).clip(min=1)
            phy_load = c[layer][phy2log[layer]] / reps[phy2log[layer]]
            per = phy_load.reshape(a.num_devices, -1).sum(-1)
            after.append(per.max() / max(per.mean(), 1e-9))
        print(f"before: mean device max/mean {before.mean():.3f}")
        print(f"after : mean device max/mean {float(np.mean(after)):.3f} with {num_phy} physical experts")
    if a.csv:
        c = counts.reshape(-1, *counts.shape[-2:]).sum(0)
        np.savetxt(a.csv, c, delimiter=",", fmt="%.0f")
    return 0


if __name__ == "__main__":
    sys.exit(main())
