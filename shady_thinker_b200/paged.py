"""Paged KV cache for one layer of a batch: a pool of fixed-size pages shared by all sequences and a page
table per sequence (``shady_kv_cache.d_page_table``).

The reference reserves ``max_seq_len`` rows per layer when the model is built (model.rs:241-256) and cannot grow
(main.rs:21, chat.rs:487).  Here a sequence holds only the pages its rows occupy, grows a page at a time and gives
its pages back when it ends, so a ragged batch needs memory for the rows it has, not for the longest possible
sequence times the batch.  The kernels take the page number of every 16-row block from the table.
"""
from __future__ import annotations

import numpy as np

from . import ops
from ._lib import F16
from .gpu import GpuContext

_ESZ = {0: 4, 1: 2, 2: 2}


class PagedKvCache:
    def __init__(self, gpu: GpuContext, *, num_seqs: int, num_pages: int, page_rows: int, num_kv_heads: int,
                 head_dim: int, kv_dtype: int = F16, max_pages_per_seq: int | None = None):
        if page_rows <= 0 or page_rows % 16:
            raise ValueError("page_rows must be a positive multiple of 16")
        if kv_dtype == 0:
            raise ValueError("paged caches are 16-bit")
        self.gpu, self.S, self.page_rows, self.num_pages = gpu, num_seqs, page_rows, num_pages
        self.nkv, self.hd, self.kv_dtype = num_kv_heads, head_dim, kv_dtype
        self.max_pages = max_pages_per_seq or num_pages
        self.page_bytes = page_rows * num_kv_heads * head_dim * _ESZ[kv_dtype]
        self.k_pool = gpu.create_storage_buffer("k_pool", num_pages * self.page_bytes)
        self.v_pool = gpu.create_storage_buffer("v_pool", num_pages * self.page_bytes)
        self.table = np.zeros((num_seqs, self.max_pages), np.uint32)
        self.d_table = gpu.upload_buffer("page_table", self.table.tobytes())
        self.pages_of = [0] * num_seqs              # pages each sequence holds
        self.free = list(range(num_pages - 1, -1, -1))

    @property
    def view(self) -> ops.KvCacheView:
        return ops.KvCacheView(self.kv_dtype, self.k_pool, self.v_pool, 0, None, None, self.d_table, self.page_rows,
                               self.max_pages)

    def ensure(self, seq: int, rows: int) -> None:
        """Give sequence ``seq`` enough pages for ``rows`` rows (uploads its table row if it changed)."""
        need = (rows + self.page_rows - 1) // self.page_rows
        if need > self.max_pages:
            raise IndexError("sequence needs more pages than max_pages_per_seq")
        have = self.pages_of[seq]
        if need <= have:
            return
        if need - have > len(self.free):
            raise MemoryError("page pool exhausted")
        for i in range(have, need):
            self.table[seq, i] = self.free.pop()
        self.pages_of[seq] = need
        self.gpu.write_buffer(self.d_table, seq * self.max_pages * 4, self.table[seq].tobytes())

    def release(self, seq: int) -> None:
        """Return the pages of a finished sequence to the pool."""
        for i in range(self.pages_of[seq]):
            self.free.append(int(self.table[seq, i]))
        self.pages_of[seq] = 0

    def row_offset(self, seq: int, row: int) -> int:
        """Element offset of cache row ``row`` of ``seq`` inside a pool (host-side bookkeeping and tests)."""
        page = int(self.table[seq, row // self.page_rows])
        return (page * self.page_rows + row % self.page_rows) * self.nkv * self.hd
