"""Fused tensor-parallel communication context.

Owns the symmetric buffers (allocated through `torch.distributed._symmetric_memory`, which
exchanges the peer mappings) and launches the kernels of `csrc/comm.cu` on them:

* `gemm_allreduce_add_rmsnorm`: the row-parallel GEMM writes its partial product straight into
  this rank's symmetric buffer, then one kernel does reduce-scatter over token rows by peer
  loads + residual add + RMSNorm + all-gather by peer stores.  The residual stream stays
  token-sharded (rank r keeps rows of its slice up to date), which is the RS -> norm -> AG
  dataflow the reference reaches with `--enable-sequence-parallel`
  (`python/sgl_jax/srt/utils/parallel_utils.py:8-51`).
* `argmax_gather`: vocab-parallel greedy sampling without gathering logits.
* `logits_gather`: vocab-parallel logits gather by peer stores (sampling with temperature / top-k / top-p
  needs the whole row), reference `python/sgl_jax/srt/layers/logits_processor.py:523`.

NCCL (`parallel/state.py`) remains the fallback for every op, and the A/B baseline.
"""

from __future__ import annotations

import ctypes
import logging

import torch

from ..ops import native

logger = logging.getLogger(__name__)


class _Symm:
    """One symmetric allocation: local tensor + device pointers of every rank's copy."""

    def __init__(self, numel: int, dtype, device, group):
        import torch.distributed._symmetric_memory as symm_mem
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        ptrs = list(self.handle.buffer_ptrs)
        self.ptrs = (ctypes.c_void_p * len(ptrs))(*ptrs)
        self.world = len(ptrs)


class FusedComm:
    def __init__(self, state, hidden: int, dtype, max_tokens: int):
        self.rank = state.tp.rank
        self.world = state.tp.size
        self.hidden = hidden
        self.dtype = dtype
        self.max_tokens = max_tokens
        self.device = state.device
        group = state.tp.device_group
        L = native.lib()
        L.sglb_ar_residual_rmsnorm.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                               ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_void_p]
        L.sglb_gemm_bf16_rs.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        self.push_epilogue = True   # GEMM epilogue does the reduce-scatter sends
        L.sglb_argmax_gather.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        L.sglb_logits_gather.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_longlong, ctypes.c_int,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_void_p]
        L.sglb_comm_barrier.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_void_p]
        self.L = L
        try:
            import torch.distributed._symmetric_memory as symm_mem
            if hasattr(symm_mem, "enable_symm_mem_for_group"):
                import warnings
                with warnings.catch_warnings():
                    warnings.simplefilter("ignore")
                    symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:
            pass
        n = (max_tokens + 8) * hidden     # room for ceil(T / world) * world rows
        self.ypart = _Symm(n, dtype, self.device, group)        # row-parallel GEMM partials
        self.gathered = _Symm(n, dtype, self.device, group)     # normalised activations, all rows
        self.flags = _Symm(L.sglb_comm_flag_bytes() // 4, torch.int32, self.device, group)
        self.flags2 = _Symm(L.sglb_comm_flag_bytes() // 4, torch.int32, self.device, group)
        self.cand = _Symm(2 * self.world * 1024, torch.int32, self.device, group)   # (value, index) x world x B
        self.epochs = torch.zeros(L.sglb_comm_max_blocks(), dtype=torch.int32, device=self.device)
        self.epochs2 = torch.zeros(L.sglb_comm_max_blocks(), dtype=torch.int32, device=self.device)
        self.flags3 = _Symm(L.sglb_comm_flag_bytes() // 4, torch.int32, self.device, group)
        self.epochs3 = torch.zeros(L.sglb_comm_max_blocks(), dtype=torch.int32, device=self.device)
        self.group = group
        self.logits_full: _Symm | None = None       # [LOGITS_GATHER_ROWS, world * shard] of the logits dtype, on demand
        self.logits_full_key = None
        torch.cuda.synchronize(self.device)
        import torch.distributed as dist
        dist.barrier(group=state.tp.cpu_group)

    @classmethod
    def create(cls, state, hidden: int, dtype, max_tokens: int = 16384) -> "FusedComm":
        if dtype != torch.bfloat16:
            raise RuntimeError("fused communication kernels are bf16 only")
        if state.tp.size > 8:
            raise RuntimeError("fused communication kernels support up to 8 ranks (one NVSwitch domain)")
        return cls(state, hidden, dtype, max_tokens)

    # ------------------------------------------------------------------ GEMM -> AR -> +res -> norm
    def supports_gemm_ar_norm(self, x: torch.Tensor, out_features: int) -> bool:
        return (x.is_cuda and x.dtype == torch.bfloat16 and out_features == self.hidden
                and x.shape[0] <= self.max_tokens and x.dim() == 2)

    def partial_buffer(self, T: int) -> torch.Tensor:
        """This rank's `[T, hidden]` slot for a partial sum that `allreduce_add_rmsnorm` will reduce."""
        return self.ypart.tensor[: T * self.hidden].view(T, self.hidden)

    def gemm_allreduce_add_rmsnorm(self, x, w, residual, norm_w, eps, gemma=False):
        T, K = x.shape
        if self.push_epilogue and K % 8 == 0 and x.is_contiguous() and w.is_contiguous():
            sc = native.gemm_scratch(x.device)
            rc = self.L.sglb_gemm_bf16_rs(x.data_ptr(), w.data_ptr(), T, self.hidden, K, sc.workspace.data_ptr(),
                                          sc.bytes, sc.counters.data_ptr(), self.ypart.ptrs, self.world, self.rank,
                                          torch.cuda.current_stream().cuda_stream)
            native._check(rc, "gemm_bf16_rs")
            return self.allreduce_add_rmsnorm(T, residual, norm_w, eps, gemma, rs_mode=1)
        native.linear(x, w, None, out=self.partial_buffer(T))
        return self.allreduce_add_rmsnorm(T, residual, norm_w, eps, gemma)

    def allreduce_add_rmsnorm(self, T: int, residual, norm_w, eps, gemma=False, rs_mode: int = 0):
        H = self.hidden
        assert residual is None or (residual.is_contiguous() and residual.shape == (T, H))
        rc = self.L.sglb_ar_residual_rmsnorm(self.ypart.ptrs, self.gathered.ptrs, self.flags.ptrs,
                                             self.epochs.data_ptr(),
                                             residual.data_ptr() if residual is not None else None,
                                             norm_w.data_ptr(), T, H, self.rank, self.world, float(eps), int(gemma),
                                             rs_mode, torch.cuda.current_stream().cuda_stream)
        native._check(rc, "ar_residual_rmsnorm")
        return self.gathered.tensor[: T * H].view(T, H), residual

    # ------------------------------------------------------------------ vocab-parallel greedy pick
    def supports_argmax_gather(self, logits: torch.Tensor) -> bool:
        return logits.is_cuda and logits.dim() == 2 and logits.shape[0] <= 1024 and logits.stride(1) == 1 \
            and logits.dtype in (torch.float32, torch.bfloat16)

    def argmax_gather(self, local_logits: torch.Tensor, vocab_start: int, vocab_size: int) -> torch.Tensor:
        B, V = local_logits.shape
        out = torch.empty(B, dtype=torch.int32, device=local_logits.device)
        rc = self.L.sglb_argmax_gather(out.data_ptr(), local_logits.data_ptr(), B, V, local_logits.stride(0),
                                       local_logits.element_size(), vocab_start, vocab_size, self.cand.ptrs,
                                       self.flags2.ptrs, self.epochs2.data_ptr(), self.rank, self.world,
                                       torch.cuda.current_stream().cuda_stream)
        native._check(rc, "argmax_gather")
        return out

    LOGITS_GATHER_ROWS = 256

    def supports_logits_gather(self, logits) -> bool:
        """Decode-sized batches of bf16 / fp32 shards.  The symmetric result buffer is allocated by the first call
        (a collective over the group: every rank reaches it in the same step), never inside a graph capture."""
        if not (logits.is_cuda and logits.dim() == 2 and logits.shape[0] <= self.LOGITS_GATHER_ROWS
                and logits.stride(1) == 1 and logits.dtype in (torch.float32, torch.bfloat16)):
            return False
        key = (logits.shape[1], logits.dtype)
        if self.logits_full_key == key:
            return True
        return self.logits_full_key is None and not torch.cuda.is_current_stream_capturing()

    def logits_gather(self, local_logits: torch.Tensor) -> torch.Tensor:
        """`[B, Vp]` shard of every rank -> `[B, world * Vp]` (rank r's columns at `r * Vp`), a view of this rank's
        symmetric buffer: valid until the next call."""
        B, Vp = local_logits.shape
        key = (Vp, local_logits.dtype)
        if self.logits_full is None:
            self.logits_full = _Symm(self.LOGITS_GATHER_ROWS * self.world * Vp, local_logits.dtype, self.device,
                                     self.group)
            self.logits_full_key = key
            torch.cuda.synchronize(self.device)
        assert self.logits_full_key == key
        rc = self.L.sglb_logits_gather(local_logits.data_ptr(), B, Vp, local_logits.stride(0),
                                       local_logits.element_size(), self.logits_full.ptrs, self.flags3.ptrs,
                                       self.epochs3.data_ptr(), self.rank, self.world,
                                       torch.cuda.current_stream().cuda_stream)
        native._check(rc, "logits_gather")
        return self.logits_full.tensor[: B * self.world * Vp].view(B, self.world * Vp)

    def barrier(self, blocks: int = 1):
        rc = self.L.sglb_comm_barrier(self.flags.ptrs, self.epochs.data_ptr(), self.rank, self.world, blocks,
                                      torch.cuda.current_stream().cuda_stream)
        native._check(rc, "comm_barrier")
