"""What a LoRA compute backend provides (reference `lora/backend/`)."""

from __future__ import annotations

import dataclasses

import torch


@dataclasses.dataclass
class LoRABatchInfo:
    """Per-forward routing of tokens to adapter slots."""
    token_slots: torch.Tensor          # i32 [T]: adapter slot of every token, -1 = base model only
    scalings: torch.Tensor             # f32 [slots]
    ranks: torch.Tensor                # i32 [slots]
    has_lora: bool = False
    # tokens sorted by slot, for segment-wise execution
    order: torch.Tensor | None = None          # i64 [T_active]
    seg_slots: list | None = None              # slot of every segment
    seg_bounds: list | None = None             # [(start, end)] into `order`


class BaseLoRABackend:
    name = "base"

    def run(self, x: torch.Tensor, y: torch.Tensor, a_buf: torch.Tensor, b_bufs: list[torch.Tensor],
            out_offsets: list[int], info: LoRABatchInfo) -> torch.Tensor:
        """`y[:, off_j : off_j + out_j] += scaling * B_j[slot] (A_j[slot] x)` for every token.
        `a_buf [slots, stack*r, in]`, `b_bufs[j] [slots, out_j, r]`."""
        raise NotImplementedError
