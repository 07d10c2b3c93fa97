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


def row_linear_add_norm(lin, x, residual, norm):
    """Returns `(norm(lin(x) + residual), lin(x) + residual)`."""
    comm = ps.get_state().fused_comm
    if comm is not None and lin.tp_size > 1 and lin.bias is None and lin.lora is None and lin.qweight is None \
            and comm.supports_gemm_ar_norm(x, lin.weight):
        return comm.gemm_allreduce_add_rmsnorm(x, lin.weight, residual, norm.weight,
                                               norm.variance_epsilon, norm.gemma)
    y = lin(x)
    return norm(y, residual)


def partial_add_norm(make_partial, num_tokens: int, hidden: int, residual, norm, tp_size: int):
    """Like `row_linear_add_norm` for a block whose per-rank partial sum is produced by arbitrary
    code (an MoE layer): `make_partial(out_or_None)` must return the `[T, H]` partial, written into
    `out` when one is given."""
    comm = ps.get_state().fused_comm
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
