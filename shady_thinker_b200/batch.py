"""Batched decode step over many sequences: the generalisation of ``Model``'s per-token attention
(model.rs:723-725) to a ragged batch, one new token per sequence per step.

The reference runs one sequence; its only multi-sequence mechanism is the ``CacheSlot`` swap
(model.rs:973-1029).  Here every sequence owns a contiguous ``[capacity][nkv][hd]`` K and V
region (the reference's row layout) inside one device allocation per layer, and one call
appends + attends for the whole batch.  Device memory comes from the context's own buffer
API; host buffers passed to :meth:`step_from_host` should be pinned for asynchronous copies.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import ops
from ._lib import BF16, F8E4M3, F8E5M2, F16, F32, AppendParams, DecodeParams
from .gpu import GpuContext, _addr

_ESZ = {F32: 4, F16: 2, BF16: 2, F8E4M3: 1, F8E5M2: 1}


class BatchedDecoder:
    def __init__(self, gpu: GpuContext, *, num_seqs: int, capacities, num_heads: int, num_kv_heads: int,
                 head_dim: int, kv_dtype: int = F16, act_dtype: int | None = None, rope_theta: float = 1e6,
                 rotary_dim: int | None = None, interleaved: bool = True, eps: float = 1e-6, has_gate: bool = False,
                 num_layers: int = 1, num_splits: int = 0, qk_norm_bf16=None, k_scale: float = 0.0,
                 v_scale: float = 0.0):
        """``kv_dtype=F8E4M3`` / ``F8E5M2`` keeps the caches as 8-bit floats (``k_scale`` / ``v_scale``: value = stored *
        scale, 0 means 1); activations are then f16."""
        self.gpu, self.S, self.nh, self.nkv, self.hd = gpu, num_seqs, num_heads, num_kv_heads, head_dim
        self.kv_dtype = kv_dtype
        if act_dtype is None:
            act_dtype = F16 if kv_dtype in (F8E4M3, F8E5M2) else kv_dtype
        self.act_dtype = act_dtype
        self.theta, self.rd = rope_theta, head_dim if rotary_dim is None else rotary_dim
        self.interleaved, self.eps, self.has_gate = interleaved, eps, has_gate
        self.num_layers, self.num_splits = num_layers, num_splits
        self.qk_norm = qk_norm_bf16   # device buffer: bf16 q_norm[hd] then k_norm[hd] (model.rs:140-168), or None
        self.fused = (not os.environ.get("SHADY_NO_FUSED_APPEND") and interleaved and
                      act_dtype in ((F32, F16) if kv_dtype in (F8E4M3, F8E5M2) else (F32, kv_dtype)) and kv_dtype != F32)
        caps = np.asarray(capacities, dtype=np.int64)
        assert caps.shape == (num_seqs,)
        row = num_kv_heads * head_dim
        esz, asz = _ESZ[kv_dtype], _ESZ[self.act_dtype]
        # rows of sequence s start at row_off[s]; 16-row padding keeps every region 16-byte aligned
        padded = (caps + 15) // 16 * 16
        self.row_off = np.concatenate([[0], np.cumsum(padded)]).astype(np.int64)
        self.layer_bytes = int(self.row_off[-1]) * row * esz
        mk = gpu.create_storage_buffer
        self.k_cache = [mk(f"k_cache_{l}", self.layer_bytes) for l in range(num_layers)]
        self.v_cache = [mk(f"v_cache_{l}", self.layer_bytes) for l in range(num_layers)]
        self._ptr_bufs = []
        self.views = []
        for l in range(num_layers):
            kp = (self.k_cache[l].ptr + self.row_off[:-1] * row * esz).astype(np.uint64)
            vp = (self.v_cache[l].ptr + self.row_off[:-1] * row * esz).astype(np.uint64)
            dk, dv = gpu.upload_buffer(f"k_ptrs_{l}", kp.tobytes()), gpu.upload_buffer(f"v_ptrs_{l}", vp.tobytes())
            self._ptr_bufs += [dk, dv]
            self.views.append(ops.KvCacheView(kv_dtype, k_ptrs=dk, v_ptrs=dv, k_scale=k_scale, v_scale=v_scale))
        qrow = num_heads * head_dim * (2 if has_gate else 1)
        self.q_in = mk("q_proj_full", num_seqs * qrow * asz)
        self.k_in = mk("k_proj", num_seqs * row * asz)
        self.v_in = mk("v_proj", num_seqs * row * asz)
        self.q_rot = mk("q_proj", num_seqs * num_heads * head_dim * asz)
        self.q_gate = mk("q_gate", num_seqs * num_heads * head_dim * 4) if has_gate else None
        self.out = mk("attn_output", num_seqs * num_heads * head_dim * asz)
        self.pos = mk("positions", num_seqs * 4)
        self.lens = mk("seq_lens", num_seqs * 4)
        self.ws_bytes = ops.decode_workspace_size(head_dim=head_dim, num_kv_heads=num_kv_heads,
                                                  num_q_heads=num_heads, num_splits=num_splits, num_seqs=num_seqs)
        self.ws = mk("attn_partials", max(self.ws_bytes, 4))
        ops.decode_workspace_init(gpu, self.ws, self.ws_bytes, head_dim=head_dim, num_kv_heads=num_kv_heads,
                                  num_q_heads=num_heads, num_splits=num_splits, num_seqs=num_seqs)
        self.in_bytes = (num_seqs * qrow + 2 * num_seqs * row) * asz
        self.out_bytes = num_seqs * num_heads * head_dim * asz
        self._lens_host = (C.c_uint32 * num_seqs)()
        self._fused_calls: dict = {}
        self.set_lengths(np.zeros(num_seqs, np.uint32))

    def close(self) -> None:
        """Free every device buffer of this decoder (the context frees what is left when it is closed)."""
        bufs = self.k_cache + self.v_cache + self._ptr_bufs + [self.q_in, self.k_in, self.v_in, self.q_rot, self.q_gate,
                                                               self.out, self.pos, self.lens, self.ws]
        for b in bufs:
            if b is not None:
                self.gpu.destroy_buffer(b)
        self.k_cache, self.v_cache, self._ptr_bufs, self.views = [], [], [], []
        self.q_in = self.k_in = self.v_in = self.q_rot = self.q_gate = self.out = self.pos = self.lens = self.ws = None
        self._fused_calls.clear()

    def set_lengths(self, lens_before) -> None:
        """Rows already in each sequence's cache; the next step appends at these positions."""
        self.lens_before = np.ascontiguousarray(lens_before, dtype=np.uint32)
        self.lens_after = (self.lens_before + 1).astype(np.uint32)
        self._lens_host[:] = self.lens_after.tolist()   # the array the prepared fused calls point at
        self.gpu.write_buffer(self.pos, 0, self.lens_before.tobytes())
        self.gpu.write_buffer(self.lens, 0, self.lens_after.tobytes())

    def kv_bytes_per_step(self) -> int:
        """Algorithmic K+V bytes one step reads: sum_i L_i * nkv * hd * 2 tensors * element size, per layer."""
        return int(self.lens_after.astype(np.int64).sum()) * self.nkv * self.hd * 2 * _ESZ[self.kv_dtype] * self.num_layers

    def append(self, layer: int = 0) -> None:
        ops.kv_append_rope(self.gpu, q_proj_full=self.q_in, k_proj=self.k_in, v_proj=self.v_in, q_out=self.q_rot,
                           q_gate=self.q_gate, cache=self.views[layer], pos_start=self.pos, num_heads=self.nh,
                           num_kv_heads=self.nkv, head_dim=self.hd, rope_theta=self.theta, rotary_dim=self.rd,
                           interleaved=self.interleaved, eps=self.eps, num_seqs=self.S, tokens_per_seq=1,
                           in_dtype=self.act_dtype, q_dtype=self.act_dtype, has_gate=self.has_gate, write_k_back=False,
                           qk_norm_bf16=self.qk_norm)

    def attend(self, layer: int = 0) -> None:
        ops.attn_decode(self.gpu, q=self.q_rot, cache=self.views[layer], seq_lens=self.lens, out=self.out,
                        head_dim=self.hd, num_kv_heads=self.nkv, num_q_heads=self.nh, num_seqs=self.S,
                        num_splits=self.num_splits, seq_lens_host=self.lens_after, q_dtype=self.act_dtype,
                        out_dtype=self.act_dtype, gate=self.q_gate, workspace=self.ws, workspace_bytes=self.ws_bytes)

    def step(self, layer: int = 0) -> None:
        """Device-resident step: activations already in q_in/k_in/v_in.  16-bit and 8-bit caches take the
        single fused launch (append + attend + gate); fp32 caches the reference's sequence of calls."""
        if self.fused:
            self.step_fused(layer)
        else:
            self.append(layer)
            self.attend(layer)

    def _fused(self, layer: int, q: int, k: int, v: int, out: int) -> None:
        """One fused launch on raw addresses.  The ctypes argument list is built once per (layer, addresses) and
        reused: a decode step is short enough for per-call marshalling to show up in the host-side latency."""
        key = (layer, q, k, v, out)
        call = self._fused_calls.get(key)
        if call is None:
            ap = AppendParams(self.nh, self.nkv, self.hd, self.eps, self.theta, self.rd, self.rd // 2, self.rd // 2, 1,
                              self.S, 1, self.act_dtype, self.act_dtype, int(self.has_gate), 0, 0)
            p = DecodeParams(self.hd, self.nkv, self.nh, self.nh // self.nkv, self.num_splits, self.S, self.act_dtype,
                             self.act_dtype)
            cs = self.views[layer].c_struct()
            vp = C.c_void_p
            args = (self.gpu.handle, C.byref(ap), C.byref(p), vp(q), vp(k), vp(v),
                    vp(_addr(self.qk_norm) or None), C.byref(cs), vp(self.lens.ptr),
                    C.cast(self._lens_host, C.POINTER(C.c_uint32)), vp(out), None, vp(self.ws.ptr), self.ws_bytes)
            if len(self._fused_calls) >= 64:      # callers that keep changing buffers must not grow this without bound
                self._fused_calls.clear()
            call = self._fused_calls[key] = (args, (ap, p, cs))
        st = self.gpu._L.shady_attn_decode_append(*call[0])
        if st:
            self.gpu._check(st)

    def step_fused(self, layer: int = 0) -> None:
        self._fused(layer, self.q_in.ptr, self.k_in.ptr, self.v_in.ptr, self.out.ptr)

    def step_from_pinned(self, q_host: int, k_host: int, v_host: int, out_host: int, layer: int = 0) -> None:
        """Full step on page-locked host buffers without copies: the fused launch reads the activations from host
        memory and writes the output rows there itself (the bytes still cross the host link, inside the kernel);
        returns when the output has arrived.  Not for fp32 caches (needs the fused launch)."""
        if not self.fused:
            raise ValueError("step_from_pinned needs the fused append+attend launch (16-bit or 8-bit cache, interleaved RoPE)")
        key = (q_host, k_host, v_host, out_host)
        if getattr(self, "_pinned_key", None) != key:
            self._pinned = tuple(self.gpu.host_device_ptr(a) for a in key)
            self._pinned_key = key
        dq, dk, dv, do = self._pinned
        self._fused(layer, dq, dk, dv, do)
        self.gpu.synchronize()

    def step_from_host(self, q_host: int, k_host: int, v_host: int, out_host: int, layer: int = 0) -> None:
        """Full step with host buffers (addresses of pinned memory): H2D activations, append, attend,
        D2H output; returns when the output has arrived."""
        g, L = self.gpu, self.gpu._L
        asz = _ESZ[self.act_dtype]
        qn = self.S * self.nh * self.hd * (2 if self.has_gate else 1) * asz
        kn = self.S * self.nkv * self.hd * asz
        g._check(L.shady_buffer_write(g.handle, C.c_void_p(self.q_in.ptr), 0, C.c_void_p(q_host), qn))
        g._check(L.shady_buffer_write(g.handle, C.c_void_p(self.k_in.ptr), 0, C.c_void_p(k_host), kn))
        g._check(L.shady_buffer_write(g.handle, C.c_void_p(self.v_in.ptr), 0, C.c_void_p(v_host), kn))
        self.step(layer)
        g._check(L.shady_buffer_read(g.handle, C.c_void_p(self.out.ptr), 0, C.c_void_p(out_host), self.out_bytes))
