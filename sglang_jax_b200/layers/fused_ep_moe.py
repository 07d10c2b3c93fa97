"""Expert-parallel MoE with a token all-to-all (`--moe-backend fused`).

The reference's `FusedEPMoE` (`python/sgl_jax/srt/layers/fused_moe.py:20`, kernel
`python/sgl_jax/srt/kernels/fused_moe/v1/kernel.py:3301`) keeps the tokens sharded over the expert-parallel
devices: every device routes its own tokens, scatters each (token, expert) row to the device that holds the
expert (`:1019-1135`), runs its local experts on what it received and gathers the results back to the
tokens' owners (`:1189-1222`), which sum their top-k rows.  `EPMoE` in contrast replicates all tokens on
every device and all-reduces a dense `[T, hidden]` partial sum.

Here the same dataflow runs between the token-sharded residual stream of the fused tensor-parallel
kernels: rank r owns the rows of its slice, so

    gate + top-k on the owned rows  ->  dispatch (peer stores, `csrc/comm.cu: moe_dispatch_kernel`)
    ->  local experts: align / gather / grouped tcgen05 GEMMs on the received rows
    ->  combine (peer stores of the weighted expert outputs into the owner's k slots per token)
    ->  owner: sum of the k slots + residual -> RMSNorm -> all-gather (`ep_reduce_residual_rmsnorm_kernel`).

Without a fused-communication context (CPU, `--disable-fused-comm`) the same dataflow goes through
`all_to_all_single` of the process group: the A/B baseline and the oracle of the kernels.
"""

from __future__ import annotations

import ctypes

import torch

from ..parallel import state as ps


ENABLED = False        # set from `--moe-backend fused` / `fused_v2` by the model runner
CALLS = 0              # layer calls that took the all-to-all dataflow (tests, bench bookkeeping)


def supported(block) -> bool:
    """The block's experts are whole-expert sharded, its router is the plain `gate -> topk` pair and there
    is no shared expert (whose tensor-parallel partial sums need the dense reduction)."""
    ex = getattr(block, "experts", None)
    return (ex is not None and ex.expert_parallel and getattr(block, "shared_expert", None) is None
            and getattr(block, "shared_experts", None) is None and hasattr(block, "gate") and hasattr(block, "topk")
            and ex.activation == "silu")


def _route(block, x):
    logits = block.gate(x)
    bias = getattr(block.gate, "e_score_correction_bias", None)
    w, ids = block.topk(logits, bias) if bias is not None else block.topk(logits)
    ex = block.experts
    if ex.expert_location is not None:
        ids = ex.expert_location.logical_to_physical(ids)
    return w.float(), ids.int()


def _local_experts(ex, x_rows, ids_rows, w_rows):
    """Run this rank's experts on received rows: a batch with top-1 routing to the expert in the metadata.
    Rows whose id is negative produce zeros."""
    saved = ex.routed_experts_capturer, ex.recorder, ex.expert_location
    ex.routed_experts_capturer = ex.recorder = ex.expert_location = None
    try:
        return ex(x_rows, w_rows.view(-1, 1), ids_rows.view(-1, 1))
    finally:
        ex.routed_experts_capturer, ex.recorder, ex.expert_location = saved


# ------------------------------------------------------------------------------------------ library path
def moe_a2a_nccl(block, h_own: torch.Tensor, group) -> torch.Tensor:
    """Dispatch / experts / combine through `all_to_all_single`; returns the MoE output of the owned rows."""
    import torch.distributed as dist
    ex = block.experts
    world = group.size
    Tl, H = h_own.shape
    w, ids = _route(block, h_own)
    k = ids.shape[1]
    flat_ids = ids.reshape(-1)
    dst = torch.div(flat_ids, ex.num_local_experts, rounding_mode="floor").clamp_(0, world - 1)
    order = torch.argsort(dst, stable=True)
    send_counts = torch.bincount(dst, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group.device_group)
    sc, rc = send_counts.tolist(), recv_counts.tolist()        # host sync: the library needs the split sizes
    x_send = h_own[torch.div(order, k, rounding_mode="floor")]
    meta_send = torch.stack([flat_ids[order].float(), w.reshape(-1)[order]], dim=1)
    x_recv = torch.empty((sum(rc), H), dtype=h_own.dtype, device=h_own.device)
    meta_recv = torch.empty((sum(rc), 2), dtype=torch.float32, device=h_own.device)
    dist.all_to_all_single(x_recv, x_send.contiguous(), rc, sc, group=group.device_group)
    dist.all_to_all_single(meta_recv, meta_send.contiguous(), rc, sc, group=group.device_group)
    if x_recv.shape[0]:
        y = _local_experts(ex, x_recv, meta_recv[:, 0].int(), meta_recv[:, 1].contiguous())
    else:
        y = x_recv
    y_back = torch.empty((len(order), H), dtype=h_own.dtype, device=h_own.device)
    dist.all_to_all_single(y_back, y.contiguous(), sc, rc, group=group.device_group)
    out = torch.zeros((Tl * k, H), dtype=torch.float32, device=h_own.device)
    out[order] = y_back.float()
    return out.view(Tl, k, H).sum(1).to(h_own.dtype)


# ------------------------------------------------------------------------------------------ NVLink path
class EPAllToAll:
    """Symmetric buffers and launches of the peer-store dispatch / combine kernels (one per fused-comm context)."""

    def __init__(self, comm, top_k: int):
        from ..parallel.fused_comm import _Symm
        self.comm = comm
        self.k = top_k
        L = comm.L
        world, H = comm.world, comm.hidden
        vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.sglb_moe_dispatch.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, vp, vp, vp, vp, vp, vp]
        L.sglb_moe_recv_prepare.argtypes = [vp, vp, i, i, i, vp, vp, vp, vp, vp, vp]
        L.sglb_moe_combine_send.argtypes = [vp, vp, vp, vp, i, i, i, i, vp, vp]
        L.sglb_ep_reduce_residual_rmsnorm.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, f, i, vp]
        # a rank owns at most this many rows (slices are rounded up to whole 128-row tiles)
        self.rows_cap = (comm.max_tokens + world - 1) // world + 128
        self.cap = self.rows_cap * top_k                 # worst case: every pair of a rank goes to one peer
        g = comm.group
        dev = comm.device
        self.recv_x = _Symm(world * self.cap * H, torch.bfloat16, dev, g)
        self.recv_meta = _Symm(world * self.cap * 4, torch.int32, dev, g)
        self.recv_count = _Symm(16, torch.int32, dev, g)
        self.ret = _Symm(self.cap * H, torch.bfloat16, dev, g)
        self.flags = _Symm(L.sglb_comm_flag_bytes() // 4, torch.int32, dev, g)
        self.epochs = torch.zeros(L.sglb_comm_max_blocks(), dtype=torch.int32, device=dev)
        self.send_count = torch.zeros(16, dtype=torch.int32, device=dev)
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        self.ids = torch.empty(world * self.cap, dtype=torch.int32, device=dev)
        self.w = torch.empty(world * self.cap, dtype=torch.float32, device=dev)
        self.total = torch.zeros(1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize(dev)

    def forward(self, block, h_full: torch.Tensor, residual, norm):
        from ..ops import moe_native, native
        comm, L = self.comm, self.comm.L
        ex = block.experts
        T, H = h_full.shape
        world, rank, k = comm.world, comm.rank, self.k
        rows_per = comm.rows_per(T)
        r0, r1 = min(rank * rows_per, T), min((rank + 1) * rows_per, T)
        stream = torch.cuda.current_stream().cuda_stream
        comm.ensure_gathered()
        h_own = h_full[r0:r1]
        Tl = r1 - r0
        if Tl > 0:
            w, ids = _route(block, h_own)
            assert ids.shape[1] == k
        else:
            w = torch.empty((0, k), dtype=torch.float32, device=h_full.device)
            ids = torch.empty((0, k), dtype=torch.int32, device=h_full.device)
        # every rank knows T, hence the largest number of pairs one rank can send: the receive regions of this
        # call are that long (the buffers are sized for the largest step)
        cap = rows_per * k
        assert cap <= self.cap
        native._check(L.sglb_moe_dispatch(h_own.data_ptr() if Tl else None, ids.data_ptr(), w.data_ptr(), Tl * k, k, H,
                                          ex.num_local_experts, world, rank, cap, self.recv_x.ptrs,
                                          self.recv_meta.ptrs, self.send_count.data_ptr(), self.done.data_ptr(),
                                          self.recv_count.ptrs, stream), "moe_dispatch")
        native._check(L.sglb_moe_recv_prepare(self.flags.ptrs, self.epochs.data_ptr(), rank, world, cap,
                                              self.recv_meta.tensor.data_ptr(), self.recv_count.tensor.data_ptr(),
                                              self.ids.data_ptr(), self.w.data_ptr(), self.total.data_ptr(), stream),
                      "moe_recv_prepare")
        R = world * cap
        x_recv = self.recv_x.tensor[: R * H].view(R, H)
        pairs = R
        if ex.workspace is None or ex.workspace.max_pairs < pairs:
            ex.workspace = moe_native.MoeWorkspace(max(pairs, 2048), ex.num_local_experts, h_full.device)
        ws = ex.workspace
        # local experts on the received rows: top-1 "routing" to the expert named in each row's metadata
        moe_native.moe_align(self.ids[:R].view(R, 1), ex.expert_start, ex.num_local_experts, ws)
        xs = moe_native.moe_gather(x_recv, ws, pairs)
        row_slot = ws.row_token
        if ex.fp8:
            valid = ws.counts[0:1]
            xq, sx = native.quant_fp8_rows(xs, valid_rows=valid)
            hmid = moe_native.grouped_gemm_fp8(xq, sx, ex.w13_weight, ex.w13_scale, ws, pairs)
            aq, sa = native.quant_fp8_rows(hmid, gated=True, valid_rows=valid)
            y = moe_native.grouped_gemm_fp8(aq, sa, ex.w2_weight, ex.w2_scale, ws, pairs)
        else:
            hmid = moe_native.grouped_gemm(xs, ex.w13_weight, ws, pairs)
            y = moe_native.grouped_gemm(native.silu_and_mul(hmid), ex.w2_weight, ws, pairs)
        native._check(L.sglb_moe_combine_send(y.data_ptr(), row_slot.data_ptr(), ws.counts.data_ptr(),
                                              self.recv_meta.tensor.data_ptr(), pairs, H, cap, world,
                                              self.ret.ptrs, stream), "moe_combine_send")
        native._check(L.sglb_ep_reduce_residual_rmsnorm(
            self.ret.tensor.data_ptr(), comm.gathered.ptrs, self.flags.ptrs, self.epochs.data_ptr(),
            residual.data_ptr() if residual is not None else None, norm.weight.data_ptr(), T, H, k, rows_per, rank,
            world, float(norm.variance_epsilon), int(norm.gemma), stream), "ep_reduce_residual_rmsnorm")
        return comm.gathered.tensor[: T * H].view(T, H), residual


def moe_a2a_add_norm(block, h_full: torch.Tensor, residual, norm):
    """`(norm(moe(h) + residual), moe(h) + residual)` with the token all-to-all dataflow; `h_full` holds all
    rows on every rank (the output of the previous fused step)."""
    from .fused_block import fused_residual_enabled
    global CALLS
    CALLS += 1
    st = ps.get_state()
    ex = block.experts
    T, H = h_full.shape
    if ex.routed_experts_capturer is not None or ex.recorder is not None:
        # the capture buffers are indexed by the row of the whole batch: route all rows once for them
        w_all, ids_all = block.topk(block.gate(h_full))
        if ex.routed_experts_capturer is not None:
            ex.routed_experts_capturer.capture(ex.layer_id, ids_all)
        if ex.recorder is not None:
            ex.recorder.record(ex.layer_id, ids_all)
    comm = st.fused_comm
    if comm is not None and fused_residual_enabled() and h_full.is_cuda and T <= comm.max_tokens and H == comm.hidden:
        a2a = getattr(comm, "ep_a2a", None)
        k = block.topk.top_k
        if a2a is None or a2a.k != k:
            a2a = comm.ep_a2a = EPAllToAll(comm, k)
        return a2a.forward(block, h_full, residual, norm)
    # library collectives: equal slices, replicated residual
    group = st.tp
    world, rank = group.size, group.rank
    rows_per = (T + world - 1) // world
    pad = rows_per * world - T
    hp = torch.cat([h_full, h_full.new_zeros(pad, H)]) if pad else h_full
    y_own = moe_a2a_nccl(block, hp[rank * rows_per:(rank + 1) * rows_per].contiguous(), group)
    y = ps.all_gather(y_own, dim=0, group=group)[:T]
    return norm(y, residual)
