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

import torch
from torch import nn

from .. import ops
from ..parallel import state as ps


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
        self.num_experts = num_experts
        self.layer_id = layer_id
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
        self.w13_weight = nn.Parameter(torch.empty(self.num_local_experts, 2 * I, hidden_size, dtype=dtype),
                                       requires_grad=False)
        self.w2_weight = nn.Parameter(torch.empty(self.num_local_experts, hidden_size, I, dtype=dtype),
                                      requires_grad=False)
        self.workspace = None
        self.routed_experts_capturer = None

    def weight_loader(self, param, w, shard_id: str, expert_id: int):
        """`shard_id` in {"gate", "up", "down"}; `w` is the full `[out, in]` tensor of one expert."""
        local = expert_id - self.expert_start
        if local < 0 or local >= self.num_local_experts:
            return
        I = self.local_intermediate
        if shard_id in ("gate", "up"):
            src = w if self.expert_parallel or self.tp_size == 1 else w.narrow(0, self.tp_rank * I, I)
            param.data[local].narrow(0, 0 if shard_id == "gate" else I, I).copy_(src)
        else:
            src = w if self.expert_parallel or self.tp_size == 1 else w.narrow(1, self.tp_rank * I, I)
            param.data[local].copy_(src)

    def quantize_(self, dtype, block_size=None):
        """Round the expert weights through `dtype` with per-channel or block scales.  The values
        are stored de-quantised in the compute dtype (the grouped GEMM runs in bf16), so this
        reproduces the numerics of a quantised checkpoint without a separate kernel path."""
        from ..utils.quantization import dequantize_tensor, quantize_tensor
        gran = "block" if block_size else "per_channel"
        for p in (self.w13_weight, self.w2_weight):
            for e in range(p.shape[0]):
                q, s = quantize_tensor(p.data[e], dtype, gran, block_size)
                p.data[e].copy_(dequantize_tensor(q, s, block_size, p.dtype))
        self.quantized = True

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                add: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """Partial sum over this rank's experts / intermediate slice (`add` is folded in, e.g. the
        shared expert's partial output)."""
        if self.routed_experts_capturer is not None:
            self.routed_experts_capturer.capture(self.layer_id, topk_ids)
        if ops.use_native(x) and self.activation == "silu":
            from ..ops import moe_native
            pairs = x.shape[0] * topk_ids.shape[1]
            if self.workspace is None or self.workspace.max_pairs < pairs:
                self.workspace = moe_native.MoeWorkspace(max(pairs, 2048), self.num_local_experts, x.device)
            return moe_native.fused_experts(x, self.w13_weight, self.w2_weight, topk_weights, topk_ids,
                                            self.expert_start, self.workspace, add, out)
        if self.activation == "silu":
            y = ops.fused_experts(x, self.w13_weight, self.w2_weight, topk_weights, topk_ids, self.expert_start, None,
                                  add)
        else:
            from ..ops import reference
            y = reference.moe_forward(x, self.w13_weight, self.w2_weight, topk_weights, topk_ids, self.expert_start,
                                      act=self.activation)
            if add is not None:
                y = (y.float() + add.float()).to(y.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y


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
