"""The row-parallel "GEMM -> reduce -> +residual -> RMSNorm" step that closes both halves
of a decoder layer (o_proj and down_proj).

Under tensor parallelism this is the communication-bound point of the layer, so it is
the unit that gets fused: with a fused-communication context installed the whole step is
one pipeline of sm_100a kernels exchanging tiles over NVLink peer memory
(`parallel/fused_comm.py`); otherwise it is GEMM + NCCL all-reduce + fused add-RMSNorm.
The reference reaches the same dataflow through GSPMD-inserted all-reduces after
`o_proj` / `down_proj` (`python/sgl_jax/srt/models/qwen3.py:28-215`).
"""

from __future__ import annotations

from ..parallel import state as ps

# The fused path keeps the residual stream token-sharded: a rank only updates the rows of its own
# slice, the other rows of its `residual` tensor go stale.  That is sound only if every consumer of
# the residual inside one model forward is a fused step, so the choice is made once per forward
# (`set_fused_residual`), never per call: a layer that cannot take the fused path (a LoRA adapter), a deep-stack add, an
# auxiliary hidden-state capture or a tracer switches the whole forward to the library all-reduce.
_FUSED_RESIDUAL = True


def set_fused_residual(on: bool) -> None:
    global _FUSED_RESIDUAL
    _FUSED_RESIDUAL = bool(on)


def fused_residual_enabled() -> bool:
    return _FUSED_RESIDUAL and ps.get_state().fused_comm is not None


def row_linear_qualifies(lin) -> bool:
    """A LoRA wrapper adds a term the fused step does not know; everything else (bias, quantised
    weight) still yields a per-rank partial sum that the fused reduce accepts."""
    return lin.lora is None


def model_supports_fused_residual(model) -> bool:
    """Every row-parallel projection of the model can feed the fused reduce -> residual -> norm step."""
    from .linear import RowParallelLinear
    return all(row_linear_qualifies(m) for m in model.modules()
               if isinstance(m, RowParallelLinear) and m.tp_size > 1)


def _plain_consumer(consumer) -> bool:
    """The layer that reads the normalised rows next is a plain bf16 projection, whose GEMM can wait for the
    all-gather chunk by chunk (`FusedComm.consume_linear`)."""
    return (consumer is not None and getattr(consumer, "qweight", 1) is None and getattr(consumer, "lora", 1) is None
            and getattr(consumer, "weight", None) is not None)


def row_linear_add_norm(lin, x, residual, norm, consumer=None):
    """Returns `(norm(lin(x) + residual), lin(x) + residual)`.  `consumer`: the linear layer that will read the
    first result next, with nothing in between; when it is a plain projection the all-gather of the normalised
    rows is not waited for here but inside that projection's GEMM."""
    comm = ps.get_state().fused_comm if _FUSED_RESIDUAL else None
    if comm is not None and lin.tp_size > 1 and comm.supports_gemm_ar_norm(x, lin.out_features):
        if not row_linear_qualifies(lin):
            raise RuntimeError("the fused residual dataflow is on but a row-parallel layer carries a LoRA adapter; "
                               "`model_supports_fused_residual` must gate the forward")
        if lin.bias is None and lin.qweight is None:
            return comm.gemm_allreduce_add_rmsnorm(x, lin.weight, residual, norm.weight,
                                                   norm.variance_epsilon, norm.gemma,
                                                   defer=_plain_consumer(consumer))
        # bias (held by rank 0 only) or quantised weight: the local product is still a partial sum
        from .linear import LinearBase
        buf = comm.partial_buffer(x.shape[0])
        buf.copy_(LinearBase.forward(lin, x))
        return comm.allreduce_add_rmsnorm(x.shape[0], residual, norm.weight, norm.variance_epsilon, norm.gemma)
    y = lin(x)
    return norm(y, residual)


def partial_add_norm(make_partial, num_tokens: int, hidden: int, residual, norm, tp_size: int, block=None, x=None):
    """Like `row_linear_add_norm` for a block whose per-rank partial sum is produced by arbitrary
    code (an MoE layer): `make_partial(out_or_None)` must return the `[T, H]` partial, written into
    `out` when one is given.  With `--moe-backend fused` and a routed-expert `block` that qualifies, the
    block's input `x` goes through the token all-to-all dataflow instead (`layers/fused_ep_moe.py`)."""
    if block is not None and x is not None and tp_size > 1:
        from . import fused_ep_moe
        if fused_ep_moe.ENABLED and fused_ep_moe.supported(block):
            return fused_ep_moe.moe_a2a_add_norm(block, x, residual, norm)
    comm = ps.get_state().fused_comm if _FUSED_RESIDUAL else None
    if comm is not None and tp_size > 1 and num_tokens <= comm.max_tokens and hidden == comm.hidden:
        buf = comm.partial_buffer(num_tokens)
        y = make_partial(buf)
        if y.data_ptr() != buf.data_ptr():
            buf.copy_(y)
        return comm.allreduce_add_rmsnorm(num_tokens, residual, norm.weight, norm.variance_epsilon, norm.gemma)
    y = make_partial(None)
    if tp_size > 1:
        y = ps.all_reduce(y)
    return norm(y, residual)
