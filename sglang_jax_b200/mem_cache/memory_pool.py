"""Request→slot table and device KV pools.

Roles match the reference's `python/sgl_jax/srt/mem_cache/memory_pool.py`
(`ReqToTokenPool` :100, `MHATokenToKVPool` :496, `SWAKVPool` :768,
`MLATokenToKVPool` :1209), but the device layout is chosen for B200:

* one tensor per layer shaped ``[num_pages, 2, kv_heads, page_size, head_dim]``.
  A (page, K|V, head) tile is therefore one contiguous ``page_size*head_dim``
  block, which the attention kernels fetch with a single 1-D bulk copy
  (16-byte aligned by construction) instead of a strided gather;
* slot ``s`` lives in page ``s // page_size`` at row ``s % page_size``; page 0 is
  never handed out so slot 0 can serve as the padding target;
* the request→slot table is authoritative on the host (numpy) because the
  allocator and the radix tree run there; a device mirror of the *page* table is
  kept up to date with per-step deltas so CUDA-graph replays never rebuild it.
"""

from __future__ import annotations

import os

import numpy as np
import torch


class ReqToTokenPool:
    """Host table ``[size, max_context_len]`` of KV slot ids plus a free list of rows."""

    def __init__(self, size: int, max_context_len: int, device: str = "cpu",
                 page_size: int = 1):
        self.size = size
        self.max_context_len = max_context_len
        self.page_size = page_size
        self.device = device
        self.req_to_token = np.zeros((size, max_context_len), dtype=np.int32)
        self.free_slots = list(range(size))
        self._dirty: list[tuple[int, int, int]] = []
        # Device mirror at page granularity, row `size` is an all-zero padding row.
        self.max_pages = (max_context_len + page_size - 1) // page_size
        self.page_table = torch.zeros((size + 1, self.max_pages), dtype=torch.int32, device=device)

    def available_size(self) -> int:
        return len(self.free_slots)

    def alloc(self, need_size: int) -> list[int] | None:
        if need_size > len(self.free_slots):
            return None
        out = self.free_slots[:need_size]
        self.free_slots = self.free_slots[need_size:]
        return out

    def free(self, idx: int | list[int]):
        if isinstance(idx, (int, np.integer)):
            self.free_slots.append(int(idx))
        else:
            self.free_slots.extend(int(i) for i in idx)

    def write(self, req_idx: int, start: int, values) -> None:
        values = np.asarray(values, dtype=np.int32)
        n = len(values)
        if n == 0:
            return
        self.req_to_token[req_idx, start:start + n] = values
        ps = self.page_size
        self._dirty.append((req_idx, start // ps, (start + n - 1) // ps + 1))

    def set_one(self, req_idx: int, pos: int, value: int) -> None:
        """Record the slot of one new token (decode); only a token that opens a new page
        changes the page table."""
        self.req_to_token[req_idx, pos] = value
        if pos % self.page_size == 0:
            self._dirty.append((req_idx, pos // self.page_size, pos // self.page_size + 1))

    def read(self, req_idx: int, length: int) -> np.ndarray:
        return self.req_to_token[req_idx, :length]

    def take_page_deltas(self) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
        """Page-table entries written since the last call, as (rows, page positions, page ids);
        the device mirror is brought up to date by scattering them."""
        if not self._dirty:
            e = np.empty(0, np.int32)
            return e, e, e
        rows, pos = [], []
        for r, a, b in self._dirty:
            rows.append(np.full(b - a, r, np.int32))
            pos.append(np.arange(a, b, dtype=np.int32))
        self._dirty = []
        rows = np.concatenate(rows)
        pos = np.concatenate(pos)
        ids = (self.req_to_token[rows, pos * self.page_size] // self.page_size).astype(np.int32)
        return rows, pos, ids

    def clear(self):
        self.free_slots = list(range(self.size))
        self.req_to_token.fill(0)
        self._dirty = []
        self.page_table.zero_()


class HybridReqToTokenPool(ReqToTokenPool):
    """Adds a ledger of recurrent-state slots for hybrid (linear-attention) models
    (reference `memory_pool.py:205`)."""

    def __init__(self, size, max_context_len, device="cpu", page_size=1, recurrent_pool=None):
        super().__init__(size, max_context_len, device, page_size)
        self.recurrent_pool = recurrent_pool
        self.req_to_recurrent = np.full((size,), -1, dtype=np.int32)

    def alloc_recurrent(self, req_idx: int) -> int | None:
        slot = self.recurrent_pool.alloc(1)
        if slot is None:
            return None
        self.req_to_recurrent[req_idx] = slot[0]
        return slot[0]

    def free(self, idx):
        ids = [idx] if isinstance(idx, (int, np.integer)) else list(idx)
        for i in ids:
            s = int(self.req_to_recurrent[i])
            if s >= 0 and self.recurrent_pool is not None:
                self.recurrent_pool.free([s])
            self.req_to_recurrent[i] = -1
        super().free(idx)


class KVCache:
    """Base of the device pools; `size` counts usable token slots."""

    def __init__(self, size: int, page_size: int, dtype: torch.dtype, layer_num: int,
                 device: str, start_layer: int = 0):
        self.size = size
        self.page_size = page_size
        self.dtype = dtype
        self.layer_num = layer_num
        self.device = device
        self.start_layer = start_layer
        # +1 page: page 0 is the reserved dummy page.
        self.num_pages = (size + page_size - 1) // page_size + 1

    def get_kv_size_bytes(self) -> int:
        raise NotImplementedError

    def cell_size_bytes(self) -> int:
        raise NotImplementedError

    def move_kv(self, src_loc: torch.Tensor, dst_loc: torch.Tensor):
        """Copy the entries of token slots `src_loc` to `dst_loc` in every layer (all sources
        are read before any destination is written)."""
        self.move_kv_cache(dst_loc, src_loc)

    def move_kv_cache(self, tgt_loc: torch.Tensor, src_loc: torch.Tensor):
        for layer in range(self.layer_num):
            a, b = self.gather(layer + self.start_layer, src_loc)
            self.set_kv_buffer(layer + self.start_layer, tgt_loc, a, b)


CANARY_BYTE = 0x5A


class MHATokenToKVPool(KVCache):
    """`SGLB_KV_CANARY_PAGES=n` (a debugging aid, the stand-in for a memory checker on the pools): every layer's
    buffer is followed, in the same allocation, by `n` guard pages filled with a byte pattern.  A kernel that writes
    through a page id just past the pool lands there instead of in a neighbouring tensor, and `check_canaries()`
    (run by the scheduler's idle-time memory check) names the layer and page that were hit."""

    def __init__(self, size, page_size, dtype, head_num, head_dim, layer_num, device,
                 start_layer: int = 0, canary_pages: int | None = None):
        super().__init__(size, page_size, dtype, layer_num, device, start_layer)
        self.head_num = head_num
        self.head_dim = head_dim
        if canary_pages is None:
            canary_pages = int(os.environ.get("SGLB_KV_CANARY_PAGES", "0"))
        self.canary_pages = max(int(canary_pages), 0)
        self.kv_buffer, self._canaries = [], []
        for _ in range(layer_num):
            whole = torch.zeros((self.num_pages + self.canary_pages, 2, head_num, page_size, head_dim), dtype=dtype,
                                device=device)
            self.kv_buffer.append(whole[: self.num_pages] if self.canary_pages else whole)
            if self.canary_pages:
                guard = whole[self.num_pages:].view(torch.uint8)
                guard.fill_(CANARY_BYTE)
                self._canaries.append(guard)

    def check_canaries(self) -> None:
        """Raise if any guard page has been written (synchronises the device)."""
        for layer, guard in enumerate(self._canaries):
            bad = guard != CANARY_BYTE
            if bool(bad.any()):
                page = int(bad.view(self.canary_pages, -1).any(dim=1).nonzero()[0])
                raise RuntimeError(f"KV pool overrun: guard page {self.num_pages + page} of layer "
                                   f"{layer + self.start_layer} was written ({int(bad.sum())} bytes differ)")

    @staticmethod
    def cell_size(head_num, head_dim, layer_num, dtype) -> int:
        return 2 * head_num * head_dim * layer_num * torch.finfo(dtype).bits // 8

    def get_kv_size_bytes(self):
        return sum(b.numel() * b.element_size() for b in self.kv_buffer)

    def get_kv_buffer(self, layer_id: int) -> torch.Tensor:
        return self.kv_buffer[layer_id - self.start_layer]

    def get_key_buffer(self, layer_id):
        return self.get_kv_buffer(layer_id)[:, 0]

    def get_value_buffer(self, layer_id):
        return self.get_kv_buffer(layer_id)[:, 1]

    def set_kv_buffer(self, layer_id: int, loc: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
        """Torch reference of the fused RoPE+KV-write kernel: scatter rows
        ``k,v [T, heads, dim]`` into slots ``loc [T]``."""
        buf = self.get_kv_buffer(layer_id)
        page = (loc // self.page_size).long()
        off = (loc % self.page_size).long()
        buf[page, 0, :, off] = k.to(self.dtype)
        buf[page, 1, :, off] = v.to(self.dtype)

    def gather(self, layer_id: int, loc: torch.Tensor):
        buf = self.get_kv_buffer(layer_id)
        page = (loc // self.page_size).long()
        off = (loc % self.page_size).long()
        return buf[page, 0, :, off], buf[page, 1, :, off]

    def move_kv_cache(self, tgt_loc: torch.Tensor, src_loc: torch.Tensor):
        for layer in range(self.layer_num):
            k, v = self.gather(layer + self.start_layer, src_loc)
            self.set_kv_buffer(layer + self.start_layer, tgt_loc, k, v)

    def get_pages(self, layer_id: int, page_ids: torch.Tensor) -> torch.Tensor:
        return self.get_kv_buffer(layer_id)[page_ids.long()]

    def set_pages(self, layer_id: int, page_ids: torch.Tensor, data: torch.Tensor):
        self.get_kv_buffer(layer_id)[page_ids.long()] = data.to(self.dtype)


class SWAKVPool(KVCache):
    """Two MHA pools — one for full-attention layers, one (smaller) for
    sliding-window layers — with a slot translation table from full-pool slot ids to
    SWA-pool slot ids (reference `memory_pool.py:768-950`)."""

    def __init__(self, size, size_swa, page_size, dtype, head_num, head_dim,
                 swa_attention_layer_ids, full_attention_layer_ids, device,
                 swa_head_num=None, swa_head_dim=None):
        super().__init__(size, page_size, dtype, len(swa_attention_layer_ids) + len(full_attention_layer_ids), device)
        self.size_swa = size_swa
        self.full_pool = MHATokenToKVPool(size, page_size, dtype, head_num, head_dim,
                                          len(full_attention_layer_ids), device)
        self.swa_pool = MHATokenToKVPool(size_swa, page_size, dtype, swa_head_num or head_num,
                                         swa_head_dim or head_dim, len(swa_attention_layer_ids), device)
        self.layers_mapping: dict[int, tuple[int, bool]] = {}
        for i, l in enumerate(full_attention_layer_ids):
            self.layers_mapping[l] = (i, False)
        for i, l in enumerate(swa_attention_layer_ids):
            self.layers_mapping[l] = (i, True)
        # full slot id -> swa slot id (0 = unmapped)
        self.full_to_swa_index_mapping = torch.zeros(
            (self.full_pool.num_pages * page_size,), dtype=torch.int32, device=device)

    def get_kv_size_bytes(self):
        return self.full_pool.get_kv_size_bytes() + self.swa_pool.get_kv_size_bytes()

    def check_canaries(self) -> None:
        self.full_pool.check_canaries()
        self.swa_pool.check_canaries()

    def is_swa_layer(self, layer_id):
        return self.layers_mapping[layer_id][1]

    def translate_loc_from_full_to_swa(self, loc: torch.Tensor) -> torch.Tensor:
        return self.full_to_swa_index_mapping[loc.long()]

    def get_kv_buffer(self, layer_id):
        idx, is_swa = self.layers_mapping[layer_id]
        return (self.swa_pool if is_swa else self.full_pool).get_kv_buffer(idx)

    def set_kv_buffer(self, layer_id, loc, k, v):
        idx, is_swa = self.layers_mapping[layer_id]
        if is_swa:
            self.swa_pool.set_kv_buffer(idx, self.translate_loc_from_full_to_swa(loc), k, v)
        else:
            self.full_pool.set_kv_buffer(idx, loc, k, v)


class MLATokenToKVPool(KVCache):
    """Latent cache for absorbed MLA: per layer ``[num_pages, page_size, kv_lora_rank + rope_dim]``
    (reference `memory_pool.py:1209-1473`; there both parts are padded to 128 lanes
    for the TPU, here 512+64 = 576 bf16 = 1152 bytes per token is already 16-byte
    aligned so no padding is needed)."""

    def __init__(self, size, page_size, dtype, kv_lora_rank, qk_rope_head_dim, layer_num, device,
                 start_layer: int = 0, index_head_dim: int = 0):
        super().__init__(size, page_size, dtype, layer_num, device, start_layer)
        self.kv_lora_rank = kv_lora_rank
        self.qk_rope_head_dim = qk_rope_head_dim
        self.kv_dim = kv_lora_rank + qk_rope_head_dim
        self.kv_buffer = [
            torch.zeros((self.num_pages, page_size, self.kv_dim), dtype=dtype, device=device)
            for _ in range(layer_num)
        ]
        # sparse-attention indexer keys (one `index_head_dim` row per token and layer), addressed
        # by the same slot ids as the latent rows
        self.index_head_dim = index_head_dim
        self.index_k_buffer = [
            torch.zeros((self.num_pages * page_size, index_head_dim), dtype=dtype, device=device)
            for _ in range(layer_num)
        ] if index_head_dim else None

    @staticmethod
    def cell_size(kv_lora_rank, qk_rope_head_dim, layer_num, dtype, index_head_dim: int = 0) -> int:
        return (kv_lora_rank + qk_rope_head_dim + index_head_dim) * layer_num * torch.finfo(dtype).bits // 8

    def get_kv_size_bytes(self):
        return sum(b.numel() * b.element_size() for b in self.kv_buffer + (self.index_k_buffer or []))

    def get_index_k_buffer(self, layer_id):
        return self.index_k_buffer[layer_id - self.start_layer]

    def get_kv_buffer(self, layer_id):
        return self.kv_buffer[layer_id - self.start_layer]

    def set_kv_buffer(self, layer_id, loc, kv_c: torch.Tensor, k_pe: torch.Tensor):
        buf = self.get_kv_buffer(layer_id).view(-1, self.kv_dim)
        buf[loc.long()] = torch.cat([kv_c, k_pe], dim=-1).to(self.dtype)

    def gather(self, layer_id, loc):
        buf = self.get_kv_buffer(layer_id).view(-1, self.kv_dim)
        rows = buf[loc.long()]
        return rows[:, :self.kv_lora_rank], rows[:, self.kv_lora_rank:]


class HybridLinearKVPool(KVCache):
    """KV pool for hybrid models: only the full-attention layers own KV pages; the
    layer id is remapped to the dense index (reference `memory_pool.py:1475`)."""

    def __init__(self, size, page_size, dtype, head_num, head_dim, full_attention_layer_ids, device):
        super().__init__(size, page_size, dtype, len(full_attention_layer_ids), device)
        self.full_layer_map = {l: i for i, l in enumerate(full_attention_layer_ids)}
        self.inner = MHATokenToKVPool(size, page_size, dtype, head_num, head_dim,
                                      len(full_attention_layer_ids), device)

    def get_kv_size_bytes(self):
        return self.inner.get_kv_size_bytes()

    def get_kv_buffer(self, layer_id):
        return self.inner.get_kv_buffer(self.full_layer_map[layer_id])

    def set_kv_buffer(self, layer_id, loc, k, v):
        self.inner.set_kv_buffer(self.full_layer_map[layer_id], loc, k, v)

    def gather(self, layer_id, loc):
        return self.inner.gather(self.full_layer_map[layer_id], loc)


class MemoryPools:
    """Named bundle of the pools one model runner owns (reference `memory_pool.py:1610`)."""

    def __init__(self, **pools):
        self._pools = dict(pools)

    def __getattr__(self, name):
        try:
            return self.__dict__["_pools"][name]
        except KeyError as e:
            raise AttributeError(name) from e

    def names(self):
        return list(self._pools)
