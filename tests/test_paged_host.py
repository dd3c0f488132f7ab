"""Host bookkeeping of the paged KV cache (no GPU): page hand-out, growth, exhaustion, release, table uploads."""
import numpy as np
import pytest

from shady_thinker_b200.paged import PagedKvCache


class _Buf:
    def __init__(self, n):
        self.ptr, self.size, self.data = 0x1000, n, bytearray(n)


class _FakeGpu:
    """Stands in for GpuContext: records what would have gone to the device."""

    def __init__(self):
        self.writes = []

    def create_storage_buffer(self, label, size):
        return _Buf(size)

    def upload_buffer(self, label, data):
        b = _Buf(len(data))
        b.data[:] = data
        return b

    def write_buffer(self, buf, offset, data):
        buf.data[offset:offset + len(data)] = data
        self.writes.append((offset, len(data)))


def _table(pc):
    return np.frombuffer(bytes(pc.d_table.data), np.uint32).reshape(pc.S, pc.max_pages)


def test_pages_are_handed_out_grown_and_returned():
    gpu = _FakeGpu()
    pc = PagedKvCache(gpu, num_seqs=3, num_pages=8, page_rows=32, num_kv_heads=2, head_dim=128, kv_dtype=1,
                      max_pages_per_seq=4)
    assert pc.page_bytes == 32 * 2 * 128 * 2 and pc.k_pool.size == 8 * pc.page_bytes
    pc.ensure(0, 1)
    pc.ensure(1, 33)          # two pages
    pc.ensure(0, 32)          # still one page: nothing uploaded
    assert pc.pages_of == [1, 2, 0] and len(gpu.writes) == 2
    pc.ensure(0, 33)          # grows by one page
    used = [int(x) for s in range(3) for x in pc.table[s, :pc.pages_of[s]]]
    assert len(set(used)) == len(used) == 4 and len(pc.free) == 4
    assert np.array_equal(_table(pc), pc.table)                     # the device copy follows the host table
    assert pc.row_offset(1, 40) == (int(pc.table[1, 1]) * 32 + 8) * 2 * 128
    with pytest.raises(IndexError):
        pc.ensure(2, 4 * 32 + 1)                                     # more than max_pages_per_seq
    pc.ensure(2, 4 * 32)
    with pytest.raises(MemoryError):
        pc.ensure(1, 3 * 32)                                         # pool exhausted
    pc.release(2)
    assert len(pc.free) == 4 and pc.pages_of[2] == 0
    pc.ensure(1, 3 * 32)
    assert pc.pages_of[1] == 3


def test_bad_page_sizes_are_refused():
    for rows, dt in ((0, 1), (24, 1), (16, 0)):
        with pytest.raises(ValueError):
            PagedKvCache(_FakeGpu(), num_seqs=1, num_pages=1, page_rows=rows, num_kv_heads=1, head_dim=128, kv_dtype=dt)
