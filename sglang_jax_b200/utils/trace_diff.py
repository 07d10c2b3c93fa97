"""Compares two precision-tracer dumps layer by layer and reports where they first diverge
(reference `python/tools/trace_diff.py`).  `python -m sglang_jax_b200.utils.trace_diff a.jsonl b.jsonl`."""

from __future__ import annotations

import argparse
import json
import sys


def load(path: str) -> dict:
    recs = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            r = json.loads(line)
            recs[(r.get("forward", 0), r.get("stage", ""), r.get("name", ""), r.get("layer"))] = r
    return recs


def diff(a: dict, b: dict, rtol: float = 1e-2, keys=("mean", "std", "abs_max", "l2")) -> list[dict]:
    out = []
    for k in sorted(set(a) & set(b), key=lambda t: (t[0], t[3] if t[3] is not None else -1, t[2])):
        ra, rb = a[k], b[k]
        worst = 0.0
        for s in keys:
            if s in ra and s in rb:
                den = max(abs(ra[s]), abs(rb[s]), 1e-12)
                worst = max(worst, abs(ra[s] - rb[s]) / den)
        out.append({"key": k, "rel": worst, "ok": worst <= rtol})
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("a")
    ap.add_argument("b")
    ap.add_argument("--rtol", type=float, default=1e-2)
    args = ap.parse_args(argv)
    rows = diff(load(args.a), load(args.b), args.rtol)
    bad = [r for r in rows if not r["ok"]]
    for r in rows:
        print(f"{'OK ' if r['ok'] else 'DIFF'} rel={r['rel']:.3e} {r['key']}")
    if bad:
        print(f"first divergence: {bad[0]['key']} (rel {bad[0]['rel']:.3e}); {len(bad)}/{len(rows)} records differ")
        return 1
    print(f"{len(rows)} records agree within rtol={args.rtol}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
