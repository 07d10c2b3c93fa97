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
import os

import torch

from ..ops import native

logger = logging.getLogger(__name__)


class _Symm:
    """One symmetric allocation: local tensor + device pointers of every rank's copy."""

    def __init__(self, numel: int, dtype, device, group):
        if group is None:
            # single-rank loop-back: an ordinary allocation is its own (and only) peer
            self.tensor = torch.zeros(numel, dtype=dtype, device=device)
            self.handle = None
            self.ptrs = (ctypes.c_void_p * 1)(self.tensor.data_ptr())
            self.world = 1
            self.multicast_ptr = 0
            return
        import torch.distributed._symmetric_memory as symm_mem
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        ptrs = list(self.handle.buffer_ptrs)
        self.ptrs = (ctypes.c_void_p * len(ptrs))(*ptrs)
        self.world = len(ptrs)
        # NVSwitch multicast mapping of the same allocation (0 when the fabric offers none)
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)


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
        # one launch for GEMM -> reduce-scatter -> residual + RMSNorm -> all-gather (SGLB_FUSED_ONE_KERNEL=0 keeps the
        # GEMM-with-push-epilogue + separate reduce kernel pair)
        self.one_kernel = os.environ.get("SGLB_FUSED_ONE_KERNEL", "1") != "0"
        L.sglb_gemm_rs_norm_ag.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                           ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                           ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        L.sglb_gemm_bf16_ag.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t,
                                        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_void_p]
        L.sglb_fused_wait_gather.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                             ctypes.c_void_p]
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
            if group is not None and hasattr(symm_mem, "enable_symm_mem_for_group"):
                import warnings
                with warnings.catch_warnings():
                    warnings.simplefilter("ignore")
                    symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:
            pass
        max_tokens = min(max_tokens, L.sglb_fused_max_tokens())
        self.max_tokens = max_tokens
        n = (max_tokens + 128 * self.world + 8) * hidden     # room for world slices rounded up to whole 128-row tiles
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
        # single-launch path: epoch-valued arrival flags (symmetric), the call counter and the local tail counters
        self.fflags = _Symm(L.sglb_fused_flag_words(), torch.int32, self.device, group)
        self.fseq = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.fctrs = torch.zeros(L.sglb_fused_ctr_ints(), dtype=torch.int32, device=self.device)
        # all-gather stores through the NVSwitch multicast mapping (one multimem.st instead of `world` stores)
        self.gathered_mc = self.gathered.multicast_ptr if os.environ.get("SGLB_AG_MULTIMEM", "0") == "1" else 0
        # (tokens,) of a deferred all-gather whose arrival nobody has waited for yet
        self.pending_gather: int | None = None
        self.logits_full: _Symm | None = None       # [LOGITS_GATHER_ROWS, world * shard] of the logits dtype, on demand
        self.logits_full_key = None
        torch.cuda.synchronize(self.device)
        if group is not None:
            import torch.distributed as dist
            dist.barrier(group=state.tp.cpu_group)

    @classmethod
    def create_loopback(cls, hidden: int, device, max_tokens: int = 4096) -> "FusedComm":
        """A one-rank context on ordinary device memory: the same kernels with `world == 1` (every peer store
        lands in this GPU's own buffers, every flag wait is satisfied by this launch itself).  For single-GPU
        tests of the fused kernels; no process group is needed."""
        from types import SimpleNamespace
        st = SimpleNamespace(tp=SimpleNamespace(rank=0, size=1, device_group=None, cpu_group=None),
                             device=torch.device(device))
        return cls(st, hidden, torch.bfloat16, max_tokens)

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

    def gemm_allreduce_add_rmsnorm(self, x, w, residual, norm_w, eps, gemma=False, defer: bool = False):
        """`norm(x @ w.T summed over ranks + residual)` for all `T` rows, and the residual (rows of this rank's
        slice updated in place).  `defer`: return without waiting for the other ranks' rows; the result must then
        be consumed by `consume_linear` (or after `ensure_gathered`)."""
        T, K = x.shape
        self.ensure_gathered()
        if self.one_kernel and K % 8 == 0 and x.is_contiguous() and w.is_contiguous():
            assert residual is None or (residual.is_contiguous() and residual.shape == (T, self.hidden))
            sc = native.gemm_scratch(x.device)
            rc = self.L.sglb_gemm_rs_norm_ag(x.data_ptr(), w.data_ptr(), T, self.hidden, K, sc.workspace.data_ptr(),
                                             sc.bytes, sc.counters.data_ptr(), self.ypart.ptrs, self.gathered.ptrs,
                                             self.gathered_mc or None, self.fflags.ptrs, self.fseq.data_ptr(),
                                             self.fctrs.data_ptr(),
                                             residual.data_ptr() if residual is not None else None, norm_w.data_ptr(),
                                             float(eps), int(gemma), int(defer), self.world, self.rank,
                                             torch.cuda.current_stream().cuda_stream)
            native._check(rc, "gemm_rs_norm_ag")
            if defer:
                self.pending_gather = T
            return self.gathered.tensor[: T * self.hidden].view(T, self.hidden), residual
        if self.push_epilogue and K % 8 == 0 and x.is_contiguous() and w.is_contiguous():
            sc = native.gemm_scratch(x.device)
            rc = self.L.sglb_gemm_bf16_rs(x.data_ptr(), w.data_ptr(), T, self.hidden, K, sc.workspace.data_ptr(),
                                          sc.bytes, sc.counters.data_ptr(), self.ypart.ptrs, self.world, self.rank,
                                          torch.cuda.current_stream().cuda_stream)
            native._check(rc, "gemm_bf16_rs")
            return self.allreduce_add_rmsnorm(T, residual, norm_w, eps, gemma, rs_mode=1)
        native.linear(x, w, None, out=self.partial_buffer(T))
        return self.allreduce_add_rmsnorm(T, residual, norm_w, eps, gemma)

    def rows_per(self, T: int) -> int:
        """Token rows each rank owns (reduces, normalises, keeps the residual of) in the single-launch path."""
        out = (ctypes.c_int * 3)()
        self.L.sglb_fused_layout(T, self.world, out)
        return int(out[0])

    def ensure_gathered(self):
        """Make the stream wait for a deferred all-gather that no flag-aware consumer has picked up."""
        T = self.pending_gather
        if T is None:
            return
        self.pending_gather = None
        rc = self.L.sglb_fused_wait_gather(self.fflags.ptrs[self.rank], self.fseq.data_ptr(), T, self.world,
                                           torch.cuda.current_stream().cuda_stream)
        native._check(rc, "fused_wait_gather")

    def consume_linear(self, x: torch.Tensor, w: torch.Tensor, bias=None) -> torch.Tensor:
        """`x @ w.T (+ bias)` where `x` may be the result of a deferred fused call: the GEMM's loader then waits for
        each chunk of rows as it needs it (all-gather -> GEMM in one launch) instead of a barrier before the GEMM."""
        T = self.pending_gather
        K, N = x.shape[-1], w.shape[0]
        if (T is None or x.dim() != 2 or x.shape[0] != T or K != self.hidden or not x.is_contiguous()
                or x.data_ptr() != self.gathered.tensor.data_ptr() or N % 8 or not w.is_contiguous()
                or w.dtype != torch.bfloat16):
            self.ensure_gathered()
            return native.linear(x, w, bias)
        self.pending_gather = None
        out = torch.empty((T, N), dtype=x.dtype, device=x.device)
        sc = native.gemm_scratch(x.device)
        rc = self.L.sglb_gemm_bf16_ag(x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
                                      out.data_ptr(), T, N, K, sc.workspace.data_ptr(), sc.bytes, sc.counters.data_ptr(),
                                      self.fflags.ptrs, self.fseq.data_ptr(), self.world, self.rank,
                                      torch.cuda.current_stream().cuda_stream)
        native._check(rc, "gemm_bf16_ag")
        return out

    def allreduce_add_rmsnorm(self, T: int, residual, norm_w, eps, gemma=False, rs_mode: int = 0):
        self.ensure_gathered()
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
