"""Per-request state of the linear-attention layers of hybrid models: the short-convolution
window and the `[H, Dk, Dv]` recurrent matrix (reference
`python/sgl_jax/srt/mem_cache/recurrent_state_pool.py:77`, `copy_slots` :230).

A slot belongs to one request (`HybridReqToTokenPool` keeps the request -> slot ledger).  Slot 0 is
a scratch slot used by padding rows.  `copy_slots` clones states (copy-on-write when a prefix with
a recurrent checkpoint is shared)."""

from __future__ import annotations

import torch


def slot_bytes(num_layers: int, conv_dim: int, conv_kernel: int, num_heads: int, head_k_dim: int, head_v_dim: int,
               conv_dtype=torch.bfloat16, state_dtype=torch.float32) -> int:
    """Bytes one state slot takes over all linear-attention layers (what `RecurrentStatePool` allocates per slot)."""
    conv = conv_dim * (conv_kernel - 1) * torch.empty((), dtype=conv_dtype).element_size()
    rec = num_heads * head_k_dim * head_v_dim * torch.empty((), dtype=state_dtype).element_size()
    return num_layers * (conv + rec)


def plan_state_slots(request_slots: int, per_slot_bytes: int, available_bytes: int, max_state_size: int | None,
                     snapshot_slots: int, memory_ratio: float, sharing: bool) -> tuple[int, int]:
    """`(snapshot slots, bytes the pool will take)` (reference `model_runner_kv_cache_mixin.py`
    `handle_recurrent_cache`, `_split_state_kv_budget`).  Priority: an explicit total (`--max-recurrent-state-size`,
    request slots included); without prefix sharing no checkpoint slots at all; an explicit
    `--recurrent-snapshot-slots >= 0`; else (`-1`) the share `ratio / (1 + ratio)` of the available memory, less the
    request slots."""
    if max_state_size is not None:
        snap = max(int(max_state_size) - request_slots, 0)
    elif not sharing:
        snap = 0
    elif snapshot_slots >= 0:
        snap = int(snapshot_slots)
    else:
        if memory_ratio <= 0:
            raise ValueError(f"recurrent_state_memory_ratio={memory_ratio} is invalid for a hybrid recurrent model; "
                             f"set --recurrent-state-memory-ratio > 0")
        total = int(available_bytes * memory_ratio / (1.0 + memory_ratio)) // max(per_slot_bytes, 1)
        snap = max(total - request_slots, 0)
    return snap, (request_slots + 1 + snap) * per_slot_bytes


class RecurrentStatePool:
    def __init__(self, size: int, num_layers: int, conv_dim: int, conv_kernel: int, num_heads: int, head_k_dim: int,
                 head_v_dim: int, device: str = "cpu", conv_dtype=torch.bfloat16, state_dtype=torch.float32,
                 snapshot_slots: int = 0):
        self.size = size
        self.num_layers = num_layers
        # slots 1..size belong to request rows; `snapshot_slots` more hold prefix-cache checkpoints
        # (owned by the scheduler's unified radix cache)
        self.snapshot_slots = snapshot_slots
        n = size + 1 + snapshot_slots
        self.conv_state = torch.zeros((num_layers, n, conv_dim, conv_kernel - 1), dtype=conv_dtype, device=device)
        self.recurrent_state = torch.zeros((num_layers, n, num_heads, head_k_dim, head_v_dim), dtype=state_dtype,
                                           device=device)
        self.free_slots = list(range(1, size + 1))
        self.device = device

    def available_size(self) -> int:
        return len(self.free_slots)

    def alloc(self, n: int) -> list[int] | None:
        if n > len(self.free_slots):
            return None
        out, self.free_slots = self.free_slots[:n], self.free_slots[n:]
        self.clear_slots(out)
        return out

    def free(self, slots) -> None:
        self.free_slots.extend(int(s) for s in slots)

    def clear_slots(self, slots) -> None:
        idx = torch.as_tensor(list(slots), dtype=torch.long, device=self.conv_state.device)
        if idx.numel():
            self.conv_state[:, idx] = 0
            self.recurrent_state[:, idx] = 0

    def copy_sequence(self, pairs) -> None:
        """Run `(src, dst)` copies in order (a later copy may read what an earlier one wrote)."""
        for s, d in pairs:
            self.conv_state[:, d] = self.conv_state[:, s]
            self.recurrent_state[:, d] = self.recurrent_state[:, s]

    def copy_slots(self, src, dst) -> None:
        s = torch.as_tensor(list(src), dtype=torch.long, device=self.conv_state.device)
        d = torch.as_tensor(list(dst), dtype=torch.long, device=self.conv_state.device)
        self.conv_state[:, d] = self.conv_state[:, s]
        self.recurrent_state[:, d] = self.recurrent_state[:, s]

    def size_bytes(self) -> int:
        return self.conv_state.numel() * self.conv_state.element_size() + \
            self.recurrent_state.numel() * self.recurrent_state.element_size()

    def clear(self) -> None:
        self.free_slots = list(range(1, self.size + 1))
        self.conv_state.zero_()
        self.recurrent_state.zero_()
