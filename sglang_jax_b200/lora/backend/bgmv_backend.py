"""Batched gather matrix-vector LoRA backend.

Reference: `python/sgl_jax/srt/lora/backend/bgmv_backend.py` (an
`einsum("td,tX,Xld->tl")` over a one-hot token->adapter matrix).  Here tokens are grouped
by adapter slot: on the GPU two small sm_100a kernels do the shrink (`h = A[slot] x`) and
the expand (`y += s * B[slot] h`) with the adapter chosen per token; on the CPU every
segment is a pair of dense matmuls.
"""

from __future__ import annotations

import torch

from .base_backend import BaseLoRABackend, LoRABatchInfo


class BgmvBackend(BaseLoRABackend):
    name = "bgmv"

    def run(self, x, y, a_buf, b_bufs, out_offsets, info: LoRABatchInfo):
        if not info.has_lora:
            return y
        if x.is_cuda:
            from ... import ops
            if ops.use_native(x) and x.dtype == torch.bfloat16:
                return ops._native().lora_bgmv(x, y, a_buf, b_bufs, out_offsets, info.token_slots, info.scalings)
        return self._segments(x, y, a_buf, b_bufs, out_offsets, info)

    @staticmethod
    def _segments(x, y, a_buf, b_bufs, out_offsets, info: LoRABatchInfo):
        stack = len(b_bufs)
        r = a_buf.shape[1] // stack
        for slot, (s, e) in zip(info.seg_slots, info.seg_bounds):
            rows = info.order[s:e]
            xs = x[rows].float()
            h = xs @ a_buf[slot].float().t()                   # [n, stack*r]
            sc = float(info.scalings[slot])
            for j, (b, off) in enumerate(zip(b_bufs, out_offsets)):
                d = h[:, j * r:(j + 1) * r] @ b[slot].float().t()
                y[rows, off:off + b.shape[1]] += (sc * d).to(y.dtype)
        return y
