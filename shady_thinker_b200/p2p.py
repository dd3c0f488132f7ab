"""Row-sharded decode of one sequence across the GPUs of a box with the merge done over NVLink peer memory.

``ShardCombiner`` owns this rank's exchange buffer, shares it with the other ranks (CUDA IPC handles travel
through ``torch.distributed`` object collectives — host plumbing only) and launches the fused exchange+merge
kernel (``shady_attn_combine_p2p``).  The reference has no counterpart (it is single-device).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .gpu import Buffer, GpuContext, _addr


class ShardCombiner:
    def __init__(self, gpu: GpuContext, *, rank: int, world: int, num_heads: int, head_dim: int, group=None,
                 loopback: bool = False):
        """``loopback=True`` builds a combiner of ``world`` ranks inside ONE process on one GPU: every entry of the
        peer table is this rank's own buffer and no other rank exists, so the flags of the other ranks never
        arrive.  It exists to exercise the bounded flag wait and its status path without a second process."""
        self.gpu, self.rank, self.world, self.nh, self.hd = gpu, rank, world, num_heads, head_dim
        L = gpu._L
        n = C.c_size_t()
        st = L.shady_combine_p2p_buffer_size(world, num_heads, head_dim, C.byref(n))
        if st != _lib.OK:
            raise _lib.ShadyError(st, "combine_p2p_buffer_size")
        self.bytes = n.value
        self.buf = gpu.create_storage_buffer("p2p_exchange", self.bytes)
        gpu.write_buffer(self.buf, 0, bytes(self.bytes))          # flags start at zero
        gpu.synchronize()
        self._opened: list[int] = []
        ptrs = [0] * world
        ptrs[rank] = self.buf.ptr
        self._dist = world > 1 and not loopback
        if loopback:
            ptrs = [self.buf.ptr] * world
        if self._dist:
            import torch.distributed as dist
            h = C.create_string_buffer(64)
            gpu._check(L.shady_ipc_export(gpu.handle, C.c_void_p(self.buf.ptr), h))
            handles = [None] * world
            dist.all_gather_object(handles, bytes(h.raw), group=group)
            for r in range(world):
                if r == rank:
                    continue
                p = C.c_void_p()
                gpu._check(L.shady_ipc_open(gpu.handle, handles[r], C.byref(p)))
                ptrs[r] = p.value
                self._opened.append(p.value)
            dist.barrier(group=group)                              # every buffer is zeroed and mapped everywhere
        self.table = gpu.upload_buffer("p2p_peer_table", np.asarray(ptrs, dtype=np.uint64).tobytes())
        self.epoch = 0
        self._calls: dict = {}

    def combine(self, records, out, out_dtype: int = _lib.F32, gate=None) -> None:
        """records: this rank's [nh][hd+2] f32 (``ops.attn_decode_shard``); out: [nh][hd].  Every rank must call
        this the same number of times."""
        g = self.gpu
        g._check(g._L.shady_attn_combine_p2p(g.handle, self.world, self.rank, self.nh, self.hd, self.epoch + 1,
                                             C.c_void_p(self.table.ptr), _addr(records), _addr(out), out_dtype,
                                             _addr(gate) or None))
        self.epoch += 1      # only a call that was launched counts: a refused one must not run ahead of the peers

    def decode_and_combine(self, *, q, cache, seq_lens, seq_len_host: int, records, out, num_kv_heads: int,
                           q_dtype: int = _lib.F32, out_dtype: int = _lib.F32, gate=None, workspace=None,
                           workspace_bytes: int = 0) -> None:
        """The whole sharded step in one cooperative launch (``shady_attn_decode_shard_p2p``): decode over this
        rank's rows, grid barrier, merge of the rank's records, exchange over NVLink, merge across ranks (a shard
        of a single span keeps two launches).  Do not mix with :meth:`combine` on the same combiner (the exchange
        buffer is laid out differently)."""
        g = self.gpu
        key = (id(cache), _addr(q), _addr(seq_lens), seq_len_host, _addr(records), _addr(out), _addr(gate), _addr(workspace))
        call = self._calls.get(key)
        if call is None:     # marshal once per distinct argument set: at N >= 4 a shard's step is shorter than that takes
            p = _lib.DecodeParams(self.hd, num_kv_heads, self.nh, self.nh // num_kv_heads, 0, 1, q_dtype, _lib.F32)
            c = cache.c_struct()
            hl = (C.c_uint32 * 1)(seq_len_host)
            vp = C.c_void_p
            args = [g.handle, C.byref(p), vp(_addr(q)), C.byref(c), vp(_addr(seq_lens)), hl, self.world, self.rank, 0,
                    vp(self.table.ptr), vp(_addr(records)), vp(_addr(out)), out_dtype, vp(_addr(gate) or None),
                    vp(_addr(workspace) or None), workspace_bytes]
            if len(self._calls) >= 64:
                self._calls.clear()
            call = self._calls[key] = (args, (p, c, hl, cache))
        call[0][8] = self.epoch + 1
        st = g._L.shady_attn_decode_shard_p2p(*call[0])
        if st:
            g._check(st)
        self.epoch += 1      # only a call that was launched counts

    def close(self, group=None) -> None:
        if self._dist:
            import torch.distributed as dist
            self.gpu.synchronize()
            dist.barrier(group=group)                              # nobody still writes into a peer's buffer
        for p in self._opened:
            self.gpu._L.shady_ipc_close(self.gpu.handle, C.c_void_p(p))
        self._opened.clear()
        if self._dist:
            import torch.distributed as dist
            dist.barrier(group=group)                              # every mapping of this buffer is closed
        for b in (self.table, self.buf):
            if b is not None:
                self.gpu.destroy_buffer(b)
        self.table = self.buf = None
