"""Packed vocabulary bitmasks (reference `python/sgl_jax/srt/constrained/bitmask_ops.py`):
int32 words, bit set = token allowed."""

from __future__ import annotations

import numpy as np
import torch


def allocate_token_bitmask(batch_size: int, vocab_size: int) -> np.ndarray:
    return np.full((batch_size, (vocab_size + 31) // 32), -1, dtype=np.int32)


def fill_bitmask_from_allowed(mask: np.ndarray, row: int, allowed_ids) -> None:
    mask[row].fill(0)
    ids = np.asarray(list(allowed_ids), dtype=np.int64)
    if ids.size:
        np.bitwise_or.at(mask[row].view(np.uint32), ids // 32, (np.uint32(1) << (ids % 32).astype(np.uint32)))


def apply_token_bitmask(logits: torch.Tensor, bitmask: torch.Tensor) -> torch.Tensor:
    from ..ops.reference import apply_token_bitmask as _apply
    return _apply(logits, bitmask)


def bitmask_to_bool(mask_row: np.ndarray, vocab_size: int) -> np.ndarray:
    bits = (mask_row.view(np.uint32)[:, None] >> np.arange(32, dtype=np.uint32)) & 1
    return bits.reshape(-1)[:vocab_size].astype(bool)
