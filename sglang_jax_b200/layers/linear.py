"""Tensor-parallel linear layers.

The reference shards one `[in, out]` kernel with mesh axis names and lets GSPMD
insert the collective (`python/sgl_jax/srt/layers/linear.py:34-113`,
`MergedColumnParallelLinear` :116).  Here each rank owns its slice outright: weights
are stored `[out_local, in_local]` (the HF layout, K-major — exactly what the tcgen05
GEMM wants for its B operand), loaded pre-sharded, and the collective is explicit
(and, on the hot path, fused into the GEMM kernel — see `parallel/fused_comm.py`).
"""

from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..parallel import state as ps


def _param(*shape, dtype):
    return nn.Parameter(torch.empty(*shape, dtype=dtype), requires_grad=False)


class LinearBase(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool, dtype):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight = _param(out_features, in_features, dtype=dtype)
        self.bias = _param(out_features, dtype=dtype) if bias else None
        self.lora = None   # set by lora.layers.wrap_linear
        self.qweight = None   # utils.quantization.QuantizedWeight once the layer is quantised

    def set_quantized(self, qw):
        """Replace the dense weight by quantised storage (the dense tensor is released)."""
        self.qweight = qw
        self.weight = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.qweight is not None:
            y = self.qweight.linear(x, self.bias)
        else:
            y = ops.linear(x, self.weight, self.bias)
        if self.lora is not None:
            y = self.lora.apply(x, y)
        return y


class ReplicatedLinear(LinearBase):
    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16):
        super().__init__(in_features, out_features, bias, dtype)

    def weight_loader(self, param, w, shard_id=None):
        param.data.copy_(w)


class ColumnParallelLinear(LinearBase):
    """Output dim split over the tensor ranks; no collective."""

    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16, tp_size=None, tp_rank=None):
        self.tp_size = tp_size if tp_size is not None else ps.tp_size()
        self.tp_rank = tp_rank if tp_rank is not None else ps.tp_rank()
        assert out_features % self.tp_size == 0
        self.out_total = out_features
        super().__init__(in_features, out_features // self.tp_size, bias, dtype)

    def weight_loader(self, param, w, shard_id=None):
        n = param.shape[0]
        param.data.copy_(w.narrow(0, self.tp_rank * n, n))


class MergedColumnParallelLinear(LinearBase):
    """Several column-parallel projections sharing one input, fused into one GEMM
    (gate_proj + up_proj).  Shard `i` of the checkpoint lands at row offset
    `sum(local_sizes[:i])`."""

    def __init__(self, in_features, output_sizes: list[int], bias=False, dtype=torch.bfloat16,
                 tp_size=None, tp_rank=None):
        self.tp_size = tp_size if tp_size is not None else ps.tp_size()
        self.tp_rank = tp_rank if tp_rank is not None else ps.tp_rank()
        assert all(s % self.tp_size == 0 for s in output_sizes)
        self.output_sizes = output_sizes
        self.local_sizes = [s // self.tp_size for s in output_sizes]
        super().__init__(in_features, sum(self.local_sizes), bias, dtype)

    def weight_loader(self, param, w, shard_id: int | None = None):
        if shard_id is None:
            # checkpoint already stores the fused tensor
            offs = 0
            loff = 0
            for full, loc in zip(self.output_sizes, self.local_sizes):
                param.data.narrow(0, loff, loc).copy_(w.narrow(0, offs + self.tp_rank * loc, loc))
                offs += full
                loff += loc
            return
        loc = self.local_sizes[shard_id]
        off = sum(self.local_sizes[:shard_id])
        param.data.narrow(0, off, loc).copy_(w.narrow(0, self.tp_rank * loc, loc))


class QKVParallelLinear(LinearBase):
    """Fused q/k/v projection.  Query heads are split over ranks; KV heads are split
    when `tp <= kv_heads` and replicated otherwise (reference
    `python/sgl_jax/srt/configs/model_config.py:623-700`)."""

    def __init__(self, hidden_size, head_dim, total_num_heads, total_num_kv_heads, bias=False,
                 dtype=torch.bfloat16, tp_size=None, tp_rank=None, v_head_dim=None):
        self.tp_size = tp_size if tp_size is not None else ps.tp_size()
        self.tp_rank = tp_rank if tp_rank is not None else ps.tp_rank()
        self.head_dim = head_dim
        self.v_head_dim = v_head_dim or head_dim
        self.total_num_heads = total_num_heads
        self.total_num_kv_heads = total_num_kv_heads
        assert total_num_heads % self.tp_size == 0
        self.num_heads = total_num_heads // self.tp_size
        if self.tp_size >= total_num_kv_heads:
            assert self.tp_size % total_num_kv_heads == 0
            self.num_kv_heads = 1
            self.num_kv_head_replicas = self.tp_size // total_num_kv_heads
        else:
            assert total_num_kv_heads % self.tp_size == 0
            self.num_kv_heads = total_num_kv_heads // self.tp_size
            self.num_kv_head_replicas = 1
        self.q_size = self.num_heads * head_dim
        self.k_size = self.num_kv_heads * head_dim
        self.v_size = self.num_kv_heads * self.v_head_dim
        super().__init__(hidden_size, self.q_size + self.k_size + self.v_size, bias, dtype)

    def weight_loader(self, param, w, shard_id: str | None = None):
        if shard_id is None:
            # fused [q|k|v] checkpoint tensor
            qt = self.total_num_heads * self.head_dim
            kt = self.total_num_kv_heads * self.head_dim
            self.weight_loader(param, w.narrow(0, 0, qt), "q")
            self.weight_loader(param, w.narrow(0, qt, kt), "k")
            self.weight_loader(param, w.narrow(0, qt + kt, w.shape[0] - qt - kt), "v")
            return
        if shard_id == "q":
            off, n, idx = 0, self.q_size, self.tp_rank
        elif shard_id == "k":
            off, n, idx = self.q_size, self.k_size, self.tp_rank // self.num_kv_head_replicas
        else:
            off, n, idx = self.q_size + self.k_size, self.v_size, self.tp_rank // self.num_kv_head_replicas
        param.data.narrow(0, off, n).copy_(w.narrow(0, idx * n, n))


class RowParallelLinear(LinearBase):
    """Input dim split over the tensor ranks; output is a partial sum.  `forward`
    returns the partial when `reduce_results=False` so the caller can hand it to a fused
    GEMM→reduce kernel or reduce it together with something else."""

    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16, reduce_results=True,
                 tp_size=None, tp_rank=None):
        self.tp_size = tp_size if tp_size is not None else ps.tp_size()
        self.tp_rank = tp_rank if tp_rank is not None else ps.tp_rank()
        assert in_features % self.tp_size == 0
        self.reduce_results = reduce_results
        super().__init__(in_features // self.tp_size, out_features, bias, dtype)

    def weight_loader(self, param, w, shard_id=None):
        if param.dim() == 1:   # bias: added once, by rank 0
            param.data.copy_(w if self.tp_rank == 0 else torch.zeros_like(w))
            return
        n = param.shape[1]
        param.data.copy_(w.narrow(1, self.tp_rank * n, n))

    def forward(self, x):
        y = super().forward(x)
        if self.reduce_results and self.tp_size > 1:
            y = ps.all_reduce(y)
        return y


# The reference has a separate `QuantizedLinear` class (`layers/linear.py:198`); here any linear
# layer becomes quantised in place through `set_quantized`.
QuantizedLinear = LinearBase
