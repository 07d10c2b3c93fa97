"""Process-group bookkeeping: one process per GPU, `torch.distributed` for plumbing.

The reference drives a 2-D JAX device mesh `("data", "tensor")` from one controller
process (`python/sgl_jax/srt/utils/mesh_utils.py:9-66`) and lets GSPMD insert the
collectives.  Here every GPU has its own process; the "mesh" is a set of process
groups (tensor, data, expert) created from the world group, NCCL on GPUs and gloo
on CPU, plus a gloo side group for host-object broadcasts.
"""

from __future__ import annotations

import datetime
import os
import threading
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist


@dataclass
class GroupInfo:
    rank: int = 0
    size: int = 1
    ranks: list[int] = field(default_factory=lambda: [0])
    device_group: Any = None
    cpu_group: Any = None


@dataclass
class ParallelState:
    world_rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    device: torch.device = torch.device("cpu")
    tp: GroupInfo = field(default_factory=GroupInfo)   # tensor axis
    dp: GroupInfo = field(default_factory=GroupInfo)   # data axis (DP attention)
    ep: GroupInfo = field(default_factory=GroupInfo)   # expert axis
    world: GroupInfo = field(default_factory=GroupInfo)
    initialized: bool = False
    fused_comm: Any = None                              # parallel.fused_comm.FusedComm or None
    step_channel: Any = None                            # parallel.step_channel.StepChannel (rank 0 -> followers)


_STATE = ParallelState()
# Several single-process engines can live in one process, each on its own device (the reference's
# "multiple engines in one process" mode for RL roll-outs, `device_indexes`): an engine's scheduler thread then
# carries its own state, which wins over the process-wide one for everything that runs on that thread.
_THREAD = threading.local()


def get_state() -> ParallelState:
    return getattr(_THREAD, "state", None) or _STATE


def bind_thread_state(state: ParallelState | None) -> None:
    """Make `state` what `get_state()` returns on the calling thread (None: back to the process-wide state)."""
    _THREAD.state = state


def single_device_state(device: str = "cuda", index: int | None = None) -> ParallelState:
    """State of a one-rank engine on `device` (`cuda:index` when an index is given); nothing process-wide changes."""
    st = ParallelState()
    if device.startswith("cuda") and torch.cuda.is_available():
        st.local_rank = int(index if index is not None else 0)
        st.device = torch.device("cuda", st.local_rank)
    st.initialized = True
    return st


def tp_rank() -> int:
    return get_state().tp.rank


def tp_size() -> int:
    return get_state().tp.size


def ep_rank() -> int:
    return get_state().ep.rank


def ep_size() -> int:
    return get_state().ep.size


def _mk_group(ranks: list[int], my_rank: int, backend_dev: str | None) -> GroupInfo | None:
    dev = dist.new_group(ranks, backend=backend_dev) if backend_dev else None
    cpu = dist.new_group(ranks, backend="gloo")
    if my_rank in ranks:
        return GroupInfo(rank=ranks.index(my_rank), size=len(ranks), ranks=ranks,
                         device_group=dev if dev is not None else cpu, cpu_group=cpu)
    return None


def init_distributed(rank: int, world_size: int, device: str = "cuda", dp_size: int = 1,
                     ep_size: int = 1, init_method: str | None = None, local_rank: int | None = None,
                     timeout_s: float | None = None) -> ParallelState:
    """Create the world group and the tensor / data / expert sub-groups.

    World layout is `[dp, tensor]` row-major: ranks of one DP replica are contiguous.
    The expert axis spans the whole world (`ep_size == world_size`) or is trivial."""
    global _STATE
    st = ParallelState(world_rank=rank, world_size=world_size)
    st.local_rank = local_rank if local_rank is not None else int(os.environ.get("LOCAL_RANK", rank))
    use_cuda = device.startswith("cuda") and torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(st.local_rank)
        st.device = torch.device("cuda", st.local_rank)
    else:
        st.device = torch.device("cpu")
    if world_size > 1:
        if not dist.is_initialized():
            kw = {}
            if timeout_s:
                kw["timeout"] = datetime.timedelta(seconds=timeout_s)
            if use_cuda:
                kw["device_id"] = st.device
            dist.init_process_group(backend="nccl" if use_cuda else "gloo", rank=rank,
                                    world_size=world_size, init_method=init_method, **kw)
        dev_backend = "nccl" if use_cuda else None
        tensor = world_size // dp_size
        all_ranks = list(range(world_size))
        st.world = _mk_group(all_ranks, rank, dev_backend)
        for d in range(dp_size):
            g = _mk_group(all_ranks[d * tensor:(d + 1) * tensor], rank, dev_backend)
            if g is not None:
                st.tp = g
        if dp_size > 1:
            for t in range(tensor):
                g = _mk_group(all_ranks[t::tensor], rank, dev_backend)
                if g is not None:
                    st.dp = g
        if ep_size > 1:
            # experts span the devices of one data-parallel section (all devices when there is one section)
            assert ep_size == tensor, "expert parallelism spans all devices of a data-parallel section"
            st.ep = st.tp if dp_size > 1 else st.world
    st.initialized = True
    _STATE = st
    return st


def reset_state():
    global _STATE
    _STATE = ParallelState()


def destroy():
    if dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:
            pass
    reset_state()


# --------------------------------------------------------------------------- collectives (NCCL / gloo path)
def all_reduce(x: torch.Tensor, group: GroupInfo | None = None) -> torch.Tensor:
    g = group or get_state().tp
    if g.size == 1:
        return x
    dist.all_reduce(x, group=g.device_group)
    return x


def all_gather(x: torch.Tensor, dim: int = -1, group: GroupInfo | None = None) -> torch.Tensor:
    g = group or get_state().tp
    if g.size == 1:
        return x
    x = x.contiguous()
    flat = torch.empty((g.size * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(flat, x, group=g.device_group)
    if dim < 0:
        dim += x.dim()
    if dim == 0:
        return flat
    out = flat.view(g.size, *x.shape)
    return out.movedim(0, dim).reshape(*x.shape[:dim], g.size * x.shape[dim], *x.shape[dim + 1:])


def reduce_scatter(x: torch.Tensor, group: GroupInfo | None = None) -> torch.Tensor:
    """Sum over ranks, each rank keeps its slice of dim 0."""
    g = group or get_state().tp
    if g.size == 1:
        return x
    out = torch.empty((x.shape[0] // g.size, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x.contiguous(), group=g.device_group)
    return out


def all_to_all_single(out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits,
                      group: GroupInfo | None = None):
    g = group or get_state().ep
    if g.size == 1:
        out.copy_(inp)
        return out
    dist.all_to_all_single(out, inp, out_splits, in_splits, group=g.device_group)
    return out


def broadcast_object(obj, src: int = 0, group: GroupInfo | None = None):
    g = group or get_state().world
    if g.size == 1:
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=g.ranks[src], group=g.cpu_group)
    return box[0]


def barrier(group: GroupInfo | None = None):
    g = group or get_state().world
    if g.size > 1:
        dist.barrier(group=g.cpu_group)
