"""Per-step records of the DFLASH worker (reference
`python/sgl_jax/srt/speculative/dflash_info.py`)."""

from __future__ import annotations

import dataclasses

import numpy as np
import torch


@dataclasses.dataclass
class DFlashDraftInput:
    """State a request carries between steps: the anchor token of the next block.  The draft
    KV of the context is already materialised in the shared slots."""
    verified_id: torch.Tensor          # [B]
    block_size: int


@dataclasses.dataclass
class DFlashVerifyInput:
    draft_tokens: torch.Tensor         # [B, block] (column 0 = anchor)
    positions: torch.Tensor            # [B * block]
    prefix_lens: np.ndarray            # [B]


@dataclasses.dataclass
class DFlashVerifyOutput:
    accept_lens: np.ndarray            # [B] accepted draft tokens
    tokens: list                       # per request: accepted tokens + bonus
