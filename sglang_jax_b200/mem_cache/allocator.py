"""Host-side allocators of KV slots.

Same contracts as the reference's `python/sgl_jax/srt/mem_cache/allocator.py`
(`TokenToKVPoolAllocator` :91, `PagedTokenToKVPoolAllocator` :161 with
`alloc_extend` :268 / `alloc_decode` :325 / `free` :358, `SWATokenToKVPoolAllocator`
:412): slot ids start at ``page_size`` because page 0 is the dummy page, extend
allocations first fill the partially used last page of the prefix, and frees are
page-granular.  State is numpy; nothing here touches the device.
"""

from __future__ import annotations

import numpy as np


class BaseTokenToKVPoolAllocator:
    def __init__(self, size: int, page_size: int, kvcache=None, dp_size: int = 1):
        self.size = size
        self.page_size = page_size
        self._kvcache = kvcache
        self.dp_size = dp_size
        self.is_not_in_free_group = True
        self.free_group: list[np.ndarray] = []

    def get_kvcache(self):
        return self._kvcache

    def free_group_begin(self):
        self.is_not_in_free_group = False
        self.free_group = []

    def free_group_end(self):
        self.is_not_in_free_group = True
        if self.free_group:
            self.free(np.concatenate(self.free_group))
            self.free_group = []


class TokenToKVPoolAllocator(BaseTokenToKVPoolAllocator):
    """page_size == 1: a free list of individual slots 1..size."""

    def __init__(self, size: int, kvcache=None, dp_size: int = 1):
        super().__init__(size, 1, kvcache, dp_size)
        self.clear()

    def clear(self):
        self.free_slots = np.arange(1, self.size + 1, dtype=np.int32)
        self.is_not_in_free_group = True
        self.free_group = []

    def available_size(self, dp_rank: int = 0) -> int:
        return len(self.free_slots)

    def alloc(self, need_size: int, dp_rank: int = 0) -> np.ndarray | None:
        if need_size > len(self.free_slots):
            return None
        out = self.free_slots[:need_size]
        self.free_slots = self.free_slots[need_size:]
        return out.copy()

    def alloc_extend(self, prefix_lens, seq_lens, last_loc, extend_num_tokens, dp_rank: int = 0):
        return self.alloc(extend_num_tokens, dp_rank)

    def alloc_decode(self, seq_lens, last_loc, dp_rank: int = 0):
        return self.alloc(len(seq_lens), dp_rank)

    def free(self, free_index, dp_rank: int = 0):
        free_index = np.asarray(free_index, dtype=np.int32).ravel()
        if free_index.size == 0:
            return
        if self.is_not_in_free_group:
            self.free_slots = np.concatenate([self.free_slots, free_index])
        else:
            self.free_group.append(free_index)

    def backup_state(self):
        return self.free_slots.copy()

    def restore_state(self, state):
        self.free_slots = state


class PagedTokenToKVPoolAllocator(BaseTokenToKVPoolAllocator):
    """page_size > 1: a free list of page ids 1..num_pages; slot = page*page_size + row."""

    def __init__(self, size: int, page_size: int, kvcache=None, dp_size: int = 1):
        super().__init__(size, page_size, kvcache, dp_size)
        self.num_pages = size // page_size
        self.clear()

    def clear(self):
        self.free_pages = np.arange(1, self.num_pages + 1, dtype=np.int32)
        self.is_not_in_free_group = True
        self.free_group = []

    def available_size(self, dp_rank: int = 0) -> int:
        return len(self.free_pages) * self.page_size

    def alloc(self, need_size: int, dp_rank: int = 0) -> np.ndarray | None:
        """Allocate whole pages; `need_size` must be page aligned."""
        assert need_size % self.page_size == 0, "paged alloc() needs a page-aligned size"
        n = need_size // self.page_size
        if n > len(self.free_pages):
            return None
        pages = self.free_pages[:n]
        self.free_pages = self.free_pages[n:]
        return (pages[:, None] * self.page_size + np.arange(self.page_size, dtype=np.int32)).reshape(-1)

    def alloc_extend(self, prefix_lens, seq_lens, last_loc, extend_num_tokens, dp_rank: int = 0):
        """Slots for tokens ``prefix_len..seq_len`` of each request.

        ``last_loc[i]`` is the slot of the last prefix token (or -1): if that page
        still has free rows they are used before new pages are taken."""
        ps = self.page_size
        prefix_lens = np.asarray(prefix_lens, dtype=np.int64)
        seq_lens = np.asarray(seq_lens, dtype=np.int64)
        last_loc = np.asarray(last_loc, dtype=np.int64)
        ext = seq_lens - prefix_lens
        assert int(ext.sum()) == extend_num_tokens
        # rows available in the partially filled last page of each prefix
        room = np.where(prefix_lens % ps == 0, 0, ps - prefix_lens % ps)
        in_old = np.minimum(room, ext)
        new_pages_each = (ext - in_old + ps - 1) // ps
        need = int(new_pages_each.sum())
        if need > len(self.free_pages):
            return None
        pages = self.free_pages[:need]
        self.free_pages = self.free_pages[need:]
        out = np.empty(extend_num_tokens, dtype=np.int32)
        o = 0
        p = 0
        for i in range(len(ext)):
            e = int(ext[i])
            if e == 0:
                continue
            a = int(in_old[i])
            if a:
                out[o:o + a] = last_loc[i] + 1 + np.arange(a)
            rest = e - a
            if rest:
                npg = int(new_pages_each[i])
                slots = (pages[p:p + npg, None].astype(np.int64) * ps + np.arange(ps)).reshape(-1)[:rest]
                out[o + a:o + e] = slots
                p += npg
            o += e
        return out

    def alloc_decode(self, seq_lens, last_loc, dp_rank: int = 0):
        """One slot per request for token index ``seq_len - 1`` (``seq_lens`` already
        include the new token)."""
        ps = self.page_size
        seq_lens = np.asarray(seq_lens, dtype=np.int64)
        last_loc = np.asarray(last_loc, dtype=np.int64)
        needs_page = (seq_lens - 1) % ps == 0
        need = int(needs_page.sum())
        if need > len(self.free_pages):
            return None
        pages = self.free_pages[:need]
        self.free_pages = self.free_pages[need:]
        out = (last_loc + 1).astype(np.int32)
        out[needs_page] = pages * ps
        return out

    def free(self, free_index, dp_rank: int = 0):
        free_index = np.asarray(free_index, dtype=np.int32).ravel()
        if free_index.size == 0:
            return
        if not self.is_not_in_free_group:
            self.free_group.append(free_index)
            return
        pages = np.unique(free_index // self.page_size)
        pages = pages[pages > 0]
        self.free_pages = np.concatenate([self.free_pages, pages.astype(np.int32)])

    def backup_state(self):
        return self.free_pages.copy()

    def restore_state(self, state):
        self.free_pages = state


class PerDPAllocator:
    """`dp_size` independent allocators over disjoint pools, addressed by `dp_rank`
    (the reference threads `dp_rank` through one allocator object,
    `allocator.py:161-410`; here each rank simply owns its own instance)."""

    def __init__(self, make, dp_size: int):
        self.ranks = [make() for _ in range(dp_size)]
        self.dp_size = dp_size
        self.page_size = self.ranks[0].page_size
        self.size = self.ranks[0].size

    def __getattr__(self, name):
        def call(*a, dp_rank: int = 0, **kw):
            return getattr(self.ranks[dp_rank], name)(*a, **kw)
        return call


class SWATokenToKVPoolAllocator(BaseTokenToKVPoolAllocator):
    """Dual allocator for hybrid sliding-window models: every token gets a slot in
    the full pool and one in the (smaller) SWA pool; SWA slots of tokens that fell
    out of the window can be released early with `free_swa`."""

    def __init__(self, size: int, size_swa: int, page_size: int, kvcache=None, dp_size: int = 1):
        super().__init__(size, page_size, kvcache, dp_size)
        self.size_swa = size_swa
        mk = (lambda s: TokenToKVPoolAllocator(s)) if page_size == 1 else \
            (lambda s: PagedTokenToKVPoolAllocator(s, page_size))
        self.full_attn_allocator = mk(size)
        self.swa_attn_allocator = mk(size_swa)
        n = (size // page_size + 2) * page_size
        self.full_to_swa_index_mapping = np.zeros(n, dtype=np.int32)

    def clear(self):
        self.full_attn_allocator.clear()
        self.swa_attn_allocator.clear()
        self.full_to_swa_index_mapping.fill(0)

    def available_size(self, dp_rank: int = 0):
        return min(self.full_available_size(), self.swa_available_size())

    def full_available_size(self):
        return self.full_attn_allocator.available_size()

    def swa_available_size(self):
        return self.swa_attn_allocator.available_size()

    def _map(self, full, swa):
        self.full_to_swa_index_mapping[full] = swa
        kv = self._kvcache
        if kv is not None and hasattr(kv, "full_to_swa_index_mapping"):
            import torch
            kv.full_to_swa_index_mapping[torch.as_tensor(full, dtype=torch.long)] = \
                torch.as_tensor(swa, dtype=torch.int32).to(kv.full_to_swa_index_mapping.device)

    def _pair(self, fn_name, *args):
        sf = self.full_attn_allocator.backup_state()
        full = getattr(self.full_attn_allocator, fn_name)(*args)
        if full is None:
            return None
        swa = getattr(self.swa_attn_allocator, fn_name)(*self._swa_args(fn_name, args))
        if swa is None:
            self.full_attn_allocator.restore_state(sf)
            return None
        self._map(full, swa)
        return full

    def _swa_args(self, fn_name, args):
        if fn_name == "alloc":
            return args
        if fn_name == "alloc_extend":
            prefix_lens, seq_lens, last_loc, n = args
            ll = np.asarray(last_loc)
            sw = np.where(ll >= 0, self.full_to_swa_index_mapping[np.maximum(ll, 0)], -1)
            return (prefix_lens, seq_lens, sw, n)
        seq_lens, last_loc = args
        ll = np.asarray(last_loc)
        return (seq_lens, self.full_to_swa_index_mapping[np.maximum(ll, 0)])

    def alloc(self, need_size, dp_rank: int = 0):
        return self._pair("alloc", need_size)

    def alloc_extend(self, prefix_lens, seq_lens, last_loc, extend_num_tokens, dp_rank: int = 0):
        return self._pair("alloc_extend", prefix_lens, seq_lens, last_loc, extend_num_tokens)

    def alloc_decode(self, seq_lens, last_loc, dp_rank: int = 0):
        return self._pair("alloc_decode", seq_lens, last_loc)

    def free(self, free_index, dp_rank: int = 0):
        free_index = np.asarray(free_index, dtype=np.int32).ravel()
        if free_index.size == 0:
            return
        self.full_attn_allocator.free(free_index)
        self.free_swa(free_index)

    def free_swa(self, free_index):
        free_index = np.asarray(free_index, dtype=np.int32).ravel()
        swa = self.full_to_swa_index_mapping[free_index]
        swa = swa[swa > 0]
        if swa.size:
            self.swa_attn_allocator.free(swa)
        self.full_to_swa_index_mapping[free_index] = 0

    def translate_loc_from_full_to_swa(self, loc):
        return self.full_to_swa_index_mapping[np.asarray(loc)]

    def backup_state(self):
        return (self.full_attn_allocator.backup_state(), self.swa_attn_allocator.backup_state(),
                self.full_to_swa_index_mapping.copy())

    def restore_state(self, st):
        self.full_attn_allocator.restore_state(st[0])
        self.swa_attn_allocator.restore_state(st[1])
        self.full_to_swa_index_mapping = st[2]
