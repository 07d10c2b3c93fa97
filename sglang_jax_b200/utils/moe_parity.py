"""Parity check of one MoE layer: the framework's expert FFN (the kernels a server would run, bf16 or quantised)
against a plain fp32 statement of the same layer, on the layer's real checkpoint weights.

    python -m sglang_jax_b200.utils.moe_parity --model-dir <hf dir> --from-config --layer-idx 3 --num-tokens 64
    python -m sglang_jax_b200.utils.moe_parity --model-dir <hf dir> --list-keys --match 'layers\\.3\\.mlp'
    python -m sglang_jax_b200.utils.moe_parity --model-dir <hf dir> --from-config --moe-weight-dtype float8_e4m3fn

Counterpart of the reference's `python/sgl_jax/tools/moe_parity_repro.py` (one layer's weights from a local
safetensors directory, synthetic tokens, router from the checkpoint or deterministic logits, fused backend against
the per-expert one, optional weight quantisation, largest element differences, npz dump).  Here the two sides are the
grouped-GEMM path of `layers/moe.py` (sm_100a kernels on a GPU, their PyTorch restatement on CPU) and an
expert-by-expert fp32 loop; with `--moe-weight-dtype` the first side runs on quantised experts, so the report is the
quantisation error of that recipe on this layer.
"""

from __future__ import annotations

import argparse
import glob
import json
import os
import re
import sys

import numpy as np
import torch


# ------------------------------------------------------------------------------------------ checkpoint access
def weight_map(model_dir: str) -> dict[str, str]:
    """Tensor name -> safetensors file, from the index when there is one, else by opening every file."""
    idx = sorted(glob.glob(os.path.join(model_dir, "*.safetensors.index.json")))
    if idx:
        with open(idx[0], encoding="utf-8") as f:
            return {k: os.path.join(model_dir, v) for k, v in json.load(f)["weight_map"].items()}
    from safetensors import safe_open
    out = {}
    for path in sorted(glob.glob(os.path.join(model_dir, "*.safetensors"))):
        with safe_open(path, framework="pt") as f:
            for k in f.keys():
                out[k] = path
    return out


def load_tensor(wm: dict[str, str], key: str) -> torch.Tensor:
    from safetensors import safe_open
    if key not in wm:
        near = [k for k in wm if key.rsplit(".", 2)[0] in k][:8]
        raise KeyError(f"{key} is not in the checkpoint" + (f"; similar keys: {near}" if near else ""))
    with safe_open(wm[key], framework="pt") as f:
        return f.get_tensor(key)


def layer_weights(wm, prefix: str, moe_path: str, num_experts: int, gate="gate_proj", up="up_proj", down="down_proj",
                  pattern="experts.{i}"):
    """`(w13 [E, 2I, H], w2 [E, H, I], router [E, H] or None, correction bias or None)` in fp32, from per-expert
    tensors or from the fused `experts.gate_up_proj` / `experts.down_proj` pair."""
    base = f"{prefix}.{moe_path}"
    if f"{base}.experts.gate_up_proj" in wm:
        gu, dn = load_tensor(wm, f"{base}.experts.gate_up_proj").float(), load_tensor(wm, f"{base}.experts.down_proj").float()
        if gu.shape[1] != 2 * dn.shape[2]:            # stored [E, H, 2I] / [E, I, H]
            gu, dn = gu.transpose(1, 2), dn.transpose(1, 2)
        w13, w2 = gu.contiguous(), dn.contiguous()
    else:
        g, u, d = [], [], []
        for e in range(num_experts):
            p = f"{base}.{pattern.format(i=e)}"
            g.append(load_tensor(wm, f"{p}.{gate}.weight").float())
            u.append(load_tensor(wm, f"{p}.{up}.weight").float())
            d.append(load_tensor(wm, f"{p}.{down}.weight").float())
        w13, w2 = torch.stack([torch.cat([a, b], 0) for a, b in zip(g, u)]), torch.stack(d)
    router = next((load_tensor(wm, k).float() for k in (f"{base}.gate.weight", f"{base}.router.weight") if k in wm), None)
    bias = next((load_tensor(wm, k).float() for k in (f"{base}.gate.e_score_correction_bias",
                                                      f"{base}.gate.expert_bias") if k in wm), None)
    return w13, w2, router, bias


# ------------------------------------------------------------------------------------------ the two sides
def reference_experts(x, w13, w2, topk_w, topk_ids, act="silu"):
    """Expert by expert in fp32: `sum_k w_k * down_e(act(gate_e x) * up_e x)`."""
    x = x.float()
    out = torch.zeros_like(x)
    I = w2.shape[2]
    fn = torch.nn.functional.silu if act == "silu" else (lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
    for e in topk_ids.unique().tolist():
        rows, slot = (topk_ids == e).nonzero(as_tuple=True)
        h = x[rows] @ w13[e].float().T
        y = (fn(h[:, :I]) * h[:, I:]) @ w2[e].float().T
        out.index_add_(0, rows, y * topk_w[rows, slot].float().unsqueeze(1))
    return out


def framework_experts(x, w13, w2, topk_w, topk_ids, dtype, device, act="silu", weight_dtype=None, block=None):
    """The expert FFN as a server runs it: `layers.moe.FusedMoE` with the weights loaded, optionally quantised."""
    from ..layers.moe import FusedMoE
    E, I2, H = w13.shape
    with torch.device(device):
        moe = FusedMoE(E, H, I2 // 2, dtype=dtype, ep_size=1, tp_size=1, tp_rank=0, activation=act)
    moe.w13_weight.data.copy_(w13.to(moe.w13_weight.dtype) if not moe.fp8 else w13.to(dtype).to(moe.w13_weight.dtype))
    moe.w2_weight.data.copy_(w2.to(moe.w2_weight.dtype) if not moe.fp8 else w2.to(dtype).to(moe.w2_weight.dtype))
    if weight_dtype is not None:
        act_dtype = weight_dtype if weight_dtype == torch.float8_e4m3fn else None
        moe.quantize_(weight_dtype, block_size=block, activation_dtype=act_dtype)
    with torch.inference_mode():
        return moe(x.to(device, dtype), topk_w.to(device), topk_ids.to(device)).float().cpu()


def describe(a: torch.Tensor, b: torch.Tensor, rel_eps: float = 1e-6) -> dict:
    d = (a - b).abs()
    return {"max_abs": float(d.max()), "mean_abs": float(d.mean()),
            "max_rel": float((d / b.abs().clamp_min(rel_eps)).max()),
            "rel_fro": float(d.norm() / b.norm().clamp_min(rel_eps)),
            "cosine": float(torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0))}


# ------------------------------------------------------------------------------------------ CLI
def parse(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model-dir", required=True)
    ap.add_argument("--layer-idx", type=int, default=0)
    ap.add_argument("--num-experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--num-tokens", type=int, default=32)
    ap.add_argument("--act-fn", default="silu", choices=("silu", "gelu"))
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--prefix", default=None, help="default: model.layers.<layer-idx>")
    ap.add_argument("--moe-path", default="mlp")
    ap.add_argument("--source-expert-pattern", default="experts.{i}")
    ap.add_argument("--gate-name", default="gate_proj")
    ap.add_argument("--up-name", default="up_proj")
    ap.add_argument("--down-name", default="down_proj")
    ap.add_argument("--from-config", action="store_true", help="read the MoE settings from config.json")
    ap.add_argument("--use-grouped-topk", action="store_true")
    ap.add_argument("--num-groups", type=int, default=1)
    ap.add_argument("--top-k-groups", type=int, default=1)
    ap.add_argument("--renormalize-topk-logits", action="store_true")
    ap.add_argument("--routed-scaling-factor", type=float, default=None)
    ap.add_argument("--score-function", default=None, choices=("softmax", "sigmoid", "tanh"))
    ap.add_argument("--deterministic-router", action="store_true",
                    help="ignore the checkpoint's router: logits that spread the tokens evenly over the experts")
    ap.add_argument("--tokens-apply-rmsnorm", action="store_true", help="unit-RMS tokens, like the layer's real input")
    ap.add_argument("--tokens-rmsnorm-eps", type=float, default=1e-6)
    ap.add_argument("--moe-weight-dtype", default=None, help="quantise the experts: float8_e4m3fn, int8, ...")
    ap.add_argument("--quant-block", type=int, nargs=2, default=None, help="block scales, e.g. 128 128")
    ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--list-keys", action="store_true")
    ap.add_argument("--match", default=None)
    ap.add_argument("--list-limit", type=int, default=200)
    ap.add_argument("--dump-npz", default=None)
    ap.add_argument("--debug-topn", type=int, default=0)
    ap.add_argument("--debug-metric", default="abs", choices=("abs", "rel"))
    ap.add_argument("--debug-rel-eps", type=float, default=1e-6)
    ap.add_argument("--atol", type=float, default=None, help="exit 1 when max_abs exceeds this")
    return ap.parse_args(argv)


def settings_from_config(args):
    with open(os.path.join(args.model_dir, "config.json"), encoding="utf-8") as f:
        cfg = json.load(f)
    cfg = cfg.get("text_config") or cfg
    get = lambda *names, default=None: next((cfg[n] for n in names if cfg.get(n) is not None), default)
    args.num_experts = get("n_routed_experts", "num_experts", "num_local_experts", default=args.num_experts)
    args.top_k = get("num_experts_per_tok", "top_k_experts", default=args.top_k)
    args.score_function = args.score_function or get("scoring_func", "score_function", default="softmax")
    args.renormalize_topk_logits = bool(get("norm_topk_prob", default=args.renormalize_topk_logits))
    if args.routed_scaling_factor is None:
        args.routed_scaling_factor = get("routed_scaling_factor", default=None)
    ng, tg = get("n_group", default=0) or 0, get("topk_group", default=0) or 0
    if ng > 1:
        args.use_grouped_topk, args.num_groups, args.top_k_groups = True, ng, tg
    return cfg


def main(argv=None) -> int:
    args = parse(argv)
    wm = weight_map(args.model_dir)
    if args.list_keys:
        pat = re.compile(args.match) if args.match else None
        keys = [k for k in sorted(wm) if pat is None or pat.search(k)]
        for k in keys[: args.list_limit]:
            print(k)
        print(f"{len(keys)} keys" + (f" ({args.list_limit} shown)" if len(keys) > args.list_limit else ""))
        return 0
    if args.from_config:
        settings_from_config(args)
    prefix = args.prefix or f"model.layers.{args.layer_idx}"
    w13, w2, router, bias = layer_weights(wm, prefix, args.moe_path, args.num_experts, args.gate_name, args.up_name,
                                          args.down_name, args.source_expert_pattern)
    E, I2, H = w13.shape
    g = torch.Generator().manual_seed(args.seed)
    x = torch.randn(args.num_tokens, H, generator=g)
    if args.tokens_apply_rmsnorm:
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + args.tokens_rmsnorm_eps)
        norm_key = f"{prefix}.post_attention_layernorm.weight"
        if norm_key in wm:
            x = x * load_tensor(wm, norm_key).float()
    dtype = getattr(torch, args.dtype)
    x = x.to(dtype).float()                                   # both sides see the same rounded tokens
    if router is None or args.deterministic_router:
        logits = torch.full((args.num_tokens, E), -4.0)
        for k in range(args.top_k):
            logits[torch.arange(args.num_tokens), (torch.arange(args.num_tokens) * args.top_k + k) % E] = 4.0 - k
    else:
        logits = x @ router.T
    from ..layers.gate import TopK
    topk = TopK(args.top_k, args.renormalize_topk_logits, args.num_groups if args.use_grouped_topk else 0,
                args.top_k_groups if args.use_grouped_topk else 0, args.routed_scaling_factor or 1.0,
                args.score_function or "softmax")
    topk_w, topk_ids = topk(logits.float(), bias)
    topk_w, topk_ids = topk_w.float().cpu(), topk_ids.long().cpu()
    wdt = getattr(torch, args.moe_weight_dtype) if args.moe_weight_dtype else None
    want = reference_experts(x, w13, w2, topk_w, topk_ids, args.act_fn)
    got = framework_experts(x, w13, w2, topk_w, topk_ids, dtype, args.device, args.act_fn, wdt,
                            tuple(args.quant_block) if args.quant_block else None)
    rep = describe(got, want, args.debug_rel_eps)
    load = torch.bincount(topk_ids.flatten(), minlength=E)
    print(json.dumps({"layer": prefix, "experts": E, "hidden": H, "intermediate": I2 // 2, "tokens": args.num_tokens,
                      "top_k": args.top_k, "device": args.device, "dtype": args.dtype,
                      "weight_dtype": args.moe_weight_dtype, "experts_hit": int((load > 0).sum()),
                      "max_tokens_per_expert": int(load.max()), **{k: round(v, 6) for k, v in rep.items()}}))
    if args.debug_topn:
        d = (got - want).abs()
        score = d if args.debug_metric == "abs" else d / want.abs().clamp_min(args.debug_rel_eps)
        for i in score.flatten().topk(min(args.debug_topn, score.numel())).indices.tolist():
            t, c = divmod(i, H)
            print(f"  token {t} column {c}: got {got[t, c]:.6f} want {want[t, c]:.6f} experts {topk_ids[t].tolist()}")
    if args.dump_npz:
        np.savez(args.dump_npz, tokens=x.numpy(), topk_weights=topk_w.numpy(), topk_ids=topk_ids.numpy(),
                 framework=got.numpy(), reference=want.numpy())
    return int(args.atol is not None and rep["max_abs"] > args.atol)


if __name__ == "__main__":
    sys.exit(main())
