"""Routed-expert feed-forward layers.

The reference's `EPMoE` (`python/sgl_jax/srt/layers/moe.py:27-760`) views the devices as an
("expert", "tensor") mesh, replicates the tokens, lets each shard compute its local experts on all
tokens and sums over the expert axis.  Here the same two shardings exist per tensor-parallel rank:

* expert parallel (`ep_size == tp_size`): each rank holds `E / tp` whole experts;
* tensor parallel experts (`ep_size == 1`): every rank holds all experts with `I / tp` of the
  intermediate dimension.

Either way a rank produces a partial sum over the token rows, which the caller reduces together
with the residual add and RMSNorm that follow (`layers/fused_block.py`).  The expert FFN itself is
align -> gather -> grouped tcgen05 GEMM -> SiLU*mul -> grouped GEMM -> weighted combine
(`ops/moe_native.py`).
"""

from __future__ import annotations

import contextlib

import torch
from torch import nn

from .. import ops
from ..parallel import state as ps


_EXPERT_STORAGE = None
_EXPERT_BLOCK = None


@contextlib.contextmanager
def expert_storage(dtype, block_size=None):
    """Experts constructed inside the block store their weights in `dtype` (only `torch.float8_e4m3fn` changes
    anything) instead of the compute dtype; `block_size == (128, 128)` selects block scales (the DeepSeek-V3
    format) instead of per-output-channel ones."""
    global _EXPERT_STORAGE, _EXPERT_BLOCK
    prev = _EXPERT_STORAGE, _EXPERT_BLOCK
    _EXPERT_STORAGE = dtype
    _EXPERT_BLOCK = tuple(block_size) if block_size else None
    try:
        yield
    finally:
        _EXPERT_STORAGE, _EXPERT_BLOCK = prev


class MoeRuntime:
    """Expert-placement options the model runner sets before the model is built (reference flags
    `ep_num_redundant_experts`, `init_expert_location`, `enable_expert_distribution_recorder`)."""

    num_redundant: int = 0
    expert_load = None            # [layers, experts] hit counts that seed the placement, or None ("trivial")
    recorder = None               # eplb.ExpertDistributionRecorder
    dispatch_algorithm: str = "dynamic"   # `--ep-dispatch-algorithm`: how tokens pick among an expert's replicas
    num_groups: int = 1           # expert groups of group-limited routing (`n_group`)
    num_nodes: int = 1            # nodes the expert-parallel ranks span: with groups, the placement keeps a group on a node


_RUNTIME = MoeRuntime()


def configure_moe_runtime(num_redundant: int = 0, init_expert_location: str | None = "trivial", recorder=None,
                          num_groups: int = 1, num_nodes: int = 1, dispatch_algorithm: str | None = None):
    _RUNTIME.num_redundant = int(num_redundant or 0)
    _RUNTIME.dispatch_algorithm = "static" if dispatch_algorithm == "static" else "dynamic"
    _RUNTIME.num_groups, _RUNTIME.num_nodes = max(int(num_groups or 1), 1), max(int(num_nodes or 1), 1)
    _RUNTIME.expert_load = None
    if init_expert_location and init_expert_location != "trivial":
        from ..eplb.expert_location import load_expert_load
        _RUNTIME.expert_load = load_expert_load(init_expert_location)
    _RUNTIME.recorder = recorder
    return _RUNTIME


class FusedMoE(nn.Module):
    def __init__(self, num_experts: int, hidden_size: int, intermediate_size: int, dtype=torch.bfloat16,
                 ep_size: int | None = None, tp_size=None, tp_rank=None, layer_id: int = 0,
                 activation: str = "silu"):
        super().__init__()
        self.activation = activation
        self.tp_size = tp_size if tp_size is not None else ps.tp_size()
        self.tp_rank = tp_rank if tp_rank is not None else ps.tp_rank()
        ep = ep_size if ep_size is not None else ps.ep_size()
        self.expert_parallel = ep > 1 and ep == self.tp_size
        self.num_logical_experts = num_experts
        self.layer_id = layer_id
        # Redundant experts (EPLB): the router keeps choosing among the logical experts; hot ones own several
        # physical slots spread over the expert-parallel ranks and tokens are dealt over the replicas
        # (reference `eplb/expert_location.py`, `layers/gate.py:163`).
        self.expert_location = None
        if self.expert_parallel and _RUNTIME.num_redundant > 0:
            from ..eplb.expert_location import ExpertLocation
            load = _RUNTIME.expert_load
            if load is not None and layer_id < len(load) and len(load[layer_id]) == num_experts:
                self.expert_location = ExpertLocation.from_load(load[layer_id], ep, _RUNTIME.num_redundant,
                                                                num_groups=_RUNTIME.num_groups,
                                                                num_nodes=_RUNTIME.num_nodes)
            else:
                self.expert_location = ExpertLocation(num_experts, ep, _RUNTIME.num_redundant)
            self.expert_location.dispatch_algorithm = _RUNTIME.dispatch_algorithm
            num_experts = self.expert_location.num_physical
        self.recorder = _RUNTIME.recorder
        self.num_experts = num_experts
        if self.expert_parallel:
            assert num_experts % self.tp_size == 0
            self.num_local_experts = num_experts // self.tp_size
            self.expert_start = self.tp_rank * self.num_local_experts
            self.local_intermediate = intermediate_size
        else:
            assert intermediate_size % self.tp_size == 0
            self.num_local_experts = num_experts
            self.expert_start = 0
            self.local_intermediate = intermediate_size // self.tp_size
        I = self.local_intermediate
        self.workspace = None
        self.routed_experts_capturer = None
        self.dtype = dtype
        # e4m3 storage from the start (set by the loader for W8A8 per-channel recipes): the bf16 experts of a large
        # model never exist on the device; each expert is quantised as its checkpoint tensor arrives
        self.fp8 = (_EXPERT_STORAGE == torch.float8_e4m3fn and self._fp8_capable(dtype, activation, hidden_size, I))
        # 128 x 128 block scales need whole blocks per expert matrix
        self.fp8_block = bool(self.fp8 and _EXPERT_BLOCK == (128, 128) and hidden_size % 128 == 0 and I % 128 == 0)
        if self.fp8 and _EXPERT_BLOCK and not self.fp8_block:
            self.fp8 = False
        store = torch.float8_e4m3fn if self.fp8 else dtype
        self.w13_weight = nn.Parameter(torch.empty(self.num_local_experts, 2 * I, hidden_size, dtype=store),
                                       requires_grad=False)
        self.w2_weight = nn.Parameter(torch.empty(self.num_local_experts, hidden_size, I, dtype=store),
                                      requires_grad=False)
        if self.fp8:
            self._register_scales(self.w13_weight.device)
            self.quantized = True

    @staticmethod
    def _fp8_capable(dtype, activation, hidden_size, intermediate) -> bool:
        return dtype == torch.bfloat16 and activation == "silu" and hidden_size % 16 == 0 and intermediate % 16 == 0

    def _register_scales(self, device, w13_scale=None, w2_scale=None):
        """Per-expert, per-output-channel fp32 scales (buffers: they follow the module across devices and are
        not checkpoint parameters).  The default 0.02 gives dummy-initialised e4m3 values the usual weight scale."""
        E, I2, H = self.w13_weight.shape
        if getattr(self, "fp8_block", False):
            s13, s2 = (E, I2 // 128, H // 128), (E, H // 128, I2 // 2 // 128)
        else:
            s13, s2 = (E, I2), (E, H)
        self.register_buffer("w13_scale", w13_scale if w13_scale is not None
                             else torch.full(s13, 0.02, dtype=torch.float32, device=device))
        self.register_buffer("w2_scale", w2_scale if w2_scale is not None
                             else torch.full(s2, 0.02, dtype=torch.float32, device=device))

    def weight_loader(self, param, w, shard_id: str, expert_id: int):
        """`shard_id` in {"gate", "up", "down"}; `w` is the full `[out, in]` tensor of one (logical) expert."""
        if self.expert_location is not None:
            # every physical slot of the logical expert that lives on this rank gets a copy
            for phys in (self.expert_location.phy2log == expert_id).nonzero()[0].tolist():
                self._load_slot(param, w, shard_id, int(phys))
            return
        self._load_slot(param, w, shard_id, expert_id)

    def _load_slot(self, param, w, shard_id: str, expert_id: int):
        local = expert_id - self.expert_start
        if local < 0 or local >= self.num_local_experts:
            return
        I = self.local_intermediate
        if shard_id in ("gate", "up"):
            src = w if self.expert_parallel or self.tp_size == 1 else w.narrow(0, self.tp_rank * I, I)
            row0 = 0 if shard_id == "gate" else I
        else:
            src = w if self.expert_parallel or self.tp_size == 1 else w.narrow(1, self.tp_rank * I, I)
            row0 = 0
        dst = param.data[local].narrow(0, row0, src.shape[0])
        if self.fp8_block:
            from ..utils.quantization import quantize_tensor
            q, sc = quantize_tensor(src.to(dst.device), torch.float8_e4m3fn, "block", (128, 128))
            dst.copy_(q)
            scale = self.w2_scale if shard_id == "down" else self.w13_scale
            scale[local].narrow(0, row0 // 128, sc.shape[0]).copy_(sc)
        elif self.fp8:
            from ..utils.quantization import quantize_tensor
            q, sc = quantize_tensor(src.to(dst.device), torch.float8_e4m3fn, "per_channel")
            dst.copy_(q)
            scale = self.w2_scale if shard_id == "down" else self.w13_scale
            scale[local].narrow(0, row0, src.shape[0]).copy_(sc.view(-1))
        else:
            dst.copy_(src)

    def quantize_(self, dtype, block_size=None, activation_dtype=None):
        """Quantise the expert weights to `dtype` with per-channel or block scales.

        W8A8 e4m3 with per-channel scales keeps real fp8 storage (`w13_weight` / `w2_weight` become e4m3, with
        fp32 `w13_scale` / `w2_scale` buffers): the bf16 tensors are released and the forward runs the grouped
        fp8 tensor-core GEMMs with dynamic per-token activation scales.  Every other recipe stores the values
        de-quantised in the compute dtype, which reproduces the numerics of a quantised checkpoint on the bf16
        grouped GEMM."""
        from ..utils.quantization import dequantize_tensor, quantize_tensor
        if self.fp8:
            return                                            # built in fp8 storage: quantised while loading
        gran = "block" if block_size else "per_channel"
        E, I2, H = self.w13_weight.shape
        fp8_storage = (dtype == torch.float8_e4m3fn and activation_dtype == torch.float8_e4m3fn and not block_size
                       and self._fp8_capable(self.w13_weight.dtype, self.activation, H, I2 // 2))
        block_storage = (dtype == torch.float8_e4m3fn and activation_dtype in (torch.float8_e4m3fn, None)
                         and tuple(block_size or ()) == (128, 128) and H % 128 == 0 and (I2 // 2) % 128 == 0
                         and self._fp8_capable(self.w13_weight.dtype, self.activation, H, I2 // 2))
        if block_storage:
            # real block-scaled fp8 storage: the bf16 tensors are released, the forward runs the grouped
            # block-scaled tensor-core GEMM with per-token-group-128 activation scales
            scales = {}
            for name in ("w13", "w2"):
                p = getattr(self, f"{name}_weight")
                q = torch.empty(p.shape, dtype=dtype, device=p.device)
                sc = torch.empty((p.shape[0], p.shape[1] // 128, p.shape[2] // 128), dtype=torch.float32,
                                 device=p.device)
                for e in range(p.shape[0]):
                    qe, se = quantize_tensor(p.data[e], dtype, "block", (128, 128))
                    q[e].copy_(qe)
                    sc[e].copy_(se)
                setattr(self, f"{name}_weight", nn.Parameter(q, requires_grad=False))
                scales[name] = sc
            self.fp8 = self.fp8_block = True
            self._register_scales(self.w13_weight.device, scales["w13"], scales["w2"])
        elif fp8_storage:
            scales = {}
            for name in ("w13", "w2"):
                p = getattr(self, f"{name}_weight")
                q = torch.empty(p.shape, dtype=dtype, device=p.device)
                sc = torch.empty(p.shape[:2], dtype=torch.float32, device=p.device)
                for e in range(p.shape[0]):
                    qe, se = quantize_tensor(p.data[e], dtype, "per_channel")
                    q[e].copy_(qe)
                    sc[e].copy_(se.view(-1))
                setattr(self, f"{name}_weight", nn.Parameter(q, requires_grad=False))
                scales[name] = sc
            self._register_scales(self.w13_weight.device, scales["w13"], scales["w2"])
            self.fp8 = True
        else:
            for p in (self.w13_weight, self.w2_weight):
                for e in range(p.shape[0]):
                    q, s = quantize_tensor(p.data[e], dtype, gran, block_size)
                    p.data[e].copy_(dequantize_tensor(q, s, block_size, p.dtype))
        self.quantized = True

    def _bf16_weights(self):
        """Expert weights in the compute dtype (de-quantised on the fly under fp8 storage)."""
        if not self.fp8:
            return self.w13_weight, self.w2_weight
        if self.fp8_block:
            def deq(w, s):
                return (w.float() * s.repeat_interleave(128, 1).repeat_interleave(128, 2)).to(self.dtype)
            return deq(self.w13_weight, self.w13_scale), deq(self.w2_weight, self.w2_scale)
        return ((self.w13_weight.float() * self.w13_scale[..., None]).to(self.dtype),
                (self.w2_weight.float() * self.w2_scale[..., None]).to(self.dtype))

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                add: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """Partial sum over this rank's experts / intermediate slice (`add` is folded in, e.g. the
        shared expert's partial output)."""
        if self.routed_experts_capturer is not None:
            self.routed_experts_capturer.capture(self.layer_id, topk_ids)
        if self.recorder is not None:
            self.recorder.record(self.layer_id, topk_ids)
        if self.expert_location is not None:
            topk_ids = self.expert_location.logical_to_physical(topk_ids)
        if ops.use_native(x) and self.activation == "silu":
            from ..ops import moe_native
            pairs = x.shape[0] * topk_ids.shape[1]
            if self.workspace is None or self.workspace.max_pairs < pairs:
                self.workspace = moe_native.MoeWorkspace(max(pairs, 2048), self.num_local_experts, x.device)
            if self.fp8_block:
                return moe_native.fused_experts_fp8_block(x, self.w13_weight, self.w13_scale, self.w2_weight,
                                                          self.w2_scale, topk_weights, topk_ids, self.expert_start,
                                                          self.workspace, add, out)
            if self.fp8:
                return moe_native.fused_experts_fp8(x, self.w13_weight, self.w13_scale, self.w2_weight, self.w2_scale,
                                                    topk_weights, topk_ids, self.expert_start, self.workspace, add,
                                                    out)
            return moe_native.fused_experts(x, self.w13_weight, self.w2_weight, topk_weights, topk_ids,
                                            self.expert_start, self.workspace, add, out)
        if self.fp8:
            y = _fp8_reference_experts(x, self, topk_weights, topk_ids)
            if add is not None:
                y = (y.float() + add.float()).to(y.dtype)
        elif self.activation == "silu":
            y = ops.fused_experts(x, self.w13_weight, self.w2_weight, topk_weights, topk_ids, self.expert_start, None,
                                  add)
        else:
            from ..ops import reference
            y = reference.moe_forward(x, self.w13_weight, self.w2_weight, topk_weights, topk_ids, self.expert_start, act=self.activation)
            if add is not None:
                y = (y.float() + add.float()).to(y.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y


def _fp8_reference_experts(x, moe: "FusedMoE", topk_weights, topk_ids):
    """Plain PyTorch statement of the W8A8 expert FFN (per-token activation scales, per-channel weight
    scales, fp32 accumulation): the oracle of the fp8 kernels and the CPU path of fp8-stored experts."""
    from ..utils.quantization import quantize_activation
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    I = moe.local_intermediate
    block = getattr(moe, "fp8_block", False)

    def expand(s):
        return s.repeat_interleave(128, 0).repeat_interleave(128, 1)

    for e in range(moe.num_local_experts):
        tok, slot = (topk_ids == e + moe.expert_start).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        if block:
            # per-token-group-128 activation scales, 128 x 128 weight block scales
            xq, sx = quantize_activation(x[tok], torch.float8_e4m3fn, 128)
            xd = xq.float() * sx.repeat_interleave(128, 1)
            h = (xd @ (moe.w13_weight[e].float() * expand(moe.w13_scale[e])).t()).to(x.dtype).float()
            a = (torch.nn.functional.silu(h[:, :I]) * h[:, I:]).to(x.dtype)
            aq, sa = quantize_activation(a, torch.float8_e4m3fn, 128)
            ad = aq.float() * sa.repeat_interleave(128, 1)
            y = (ad @ (moe.w2_weight[e].float() * expand(moe.w2_scale[e])).t()).to(x.dtype).float()
            out.index_add_(0, tok, y * topk_weights[tok, slot].float()[:, None])
            continue
        xq, sx = quantize_activation(x[tok], torch.float8_e4m3fn)
        h = (xq.float() @ moe.w13_weight[e].float().t()) * sx * moe.w13_scale[e][None, :]
        h = h.to(x.dtype).float()
        a = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
        aq, sa = quantize_activation(a, torch.float8_e4m3fn)
        y = (aq.float() @ moe.w2_weight[e].float().t()) * sa * moe.w2_scale[e][None, :]
        y = y.to(x.dtype).float()
        out.index_add_(0, tok, y * topk_weights[tok, slot].float()[:, None])
    return out.to(x.dtype)


EPMoE = FusedMoE


def create_moe_weights_mapping(prefix: str, num_experts: int, gate="gate_proj", up="up_proj", down="down_proj"):
    """(checkpoint name) -> (param name, shard id, expert id) for per-expert HF tensors
    (reference `layers/moe.py:760`)."""
    out = {}
    for e in range(num_experts):
        out[f"{prefix}.experts.{e}.{gate}.weight"] = (f"{prefix}.experts.w13_weight", "gate", e)
        out[f"{prefix}.experts.{e}.{up}.weight"] = (f"{prefix}.experts.w13_weight", "up", e)
        out[f"{prefix}.experts.{e}.{down}.weight"] = (f"{prefix}.experts.w2_weight", "down", e)
    return out
