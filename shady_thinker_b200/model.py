"""Host-side mirror of the attention part of the reference's ``Model`` (src/model.rs).

Only the hot path is here: the buffers of ``InferenceState`` that the three private helpers
touch (model.rs:57-86, 226-256), and the helpers themselves with their reference names —
``fused_split_qknorm_kvstore`` (model.rs:486), ``gqa_attention`` (model.rs:516) and
``sigmoid_mul_gate`` (model.rs:576) — whose bodies call the CUDA backend instead of
``gpu.dispatch(wgsl…)``.  ``CacheSlot`` / ``alloc_cache_slot`` / ``swap_cache``
(model.rs:93-99, 973-1029) are mirrored for the KV part.
"""
from __future__ import annotations

import ctypes as C
import struct
from dataclasses import dataclass, field

import numpy as np

from . import ops
from ._lib import BF16, F16, F32, AppendParams, DecodeParams  # noqa: F401
from .gpu import Buffer, GpuContext

#: model.rs:89 fixes this at 1 at compile time; here it is a run-time value and 0 means
#: "pick a length-balanced split".
NUM_ATTN_SPLITS = 0


@dataclass
class ModelConfig:
    """The ``ModelConfig`` fields the hot path reads, with the reference defaults
    (src/weights.rs:93-152)."""

    num_attention_heads: int
    num_key_value_heads: int
    num_hidden_layers: int = 1
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e7
    partial_rotary_factor: float = 0.25
    mrope_interleaved: bool = True

    @property
    def rotary_dim(self) -> int:
        # model.rs:33: (config.head_dim as f32 * config.partial_rotary_factor) as u32
        return int(np.float32(self.head_dim) * np.float32(self.partial_rotary_factor))


@dataclass
class CacheSlot:
    """model.rs:93-99 (KV part)."""

    k_cache: list[Buffer]
    v_cache: list[Buffer]
    seq_len: int = 0


@dataclass
class InferenceState:
    q_out: Buffer
    q_proj: Buffer
    q_gate: Buffer
    k_out: Buffer
    v_out: Buffer
    attn_output: Buffer
    attn_partials: Buffer
    k_cache: list[Buffer]
    v_cache: list[Buffer]
    qknorm_params: list[Buffer | None]
    position: Buffer
    seq_len_dev: Buffer
    partials_bytes: int = 0
    extra: dict = field(default_factory=dict)


class Model:
    """Attention-only ``Model``: one sequence, one token per step, like the reference."""

    def __init__(self, gpu: GpuContext, config: ModelConfig, max_seq_len: int, kv_dtype: int = F32,
                 num_attn_splits: int = NUM_ATTN_SPLITS):
        self.config = config
        self.max_seq_len = max_seq_len
        self.kv_dtype = kv_dtype
        self.num_attn_splits = num_attn_splits
        self.seq_len = 0
        self._pos_on_device = self._len_on_device = None   # host copies of the two device counters
        self._len_host = (C.c_uint32 * 1)()                 # seq_lens_host of the prepared decode calls
        self._calls: dict = {}
        nh, nkv, hd, nl = (config.num_attention_heads, config.num_key_value_heads, config.head_dim,
                           config.num_hidden_layers)
        f = 4
        esz = 4 if kv_dtype == F32 else 2
        ws = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh,
                                       num_splits=num_attn_splits, num_seqs=1)
        mk = gpu.create_storage_buffer
        self.state = InferenceState(
            q_out=mk("q_out", nh * hd * 2 * f), q_proj=mk("q_proj", nh * hd * f), q_gate=mk("q_gate", nh * hd * f),
            k_out=mk("k_out", nkv * hd * f), v_out=mk("v_out", nkv * hd * f),
            attn_output=mk("attn_output", nh * hd * f), attn_partials=mk("attn_partials", max(ws, 4)),
            k_cache=[mk(f"k_cache_{i}", max_seq_len * nkv * hd * esz) for i in range(nl)],
            v_cache=[mk(f"v_cache_{i}", max_seq_len * nkv * hd * esz) for i in range(nl)],
            qknorm_params=[None] * nl, position=mk("position", 4), seq_len_dev=mk("seq_len", 4), partials_bytes=ws)
        ops.decode_workspace_init(gpu, self.state.attn_partials, ws, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh,
                                  num_splits=num_attn_splits, num_seqs=1)

    # model.rs:337-346 — the reference packs a 5,152-byte uniform; only the bf16 weights
    # (q then k) are data, the header fields travel by value here.
    def init_qknorm_params(self, gpu: GpuContext, layer_idx: int, q_norm_bytes: bytes, k_norm_bytes: bytes) -> None:
        hd = self.config.head_dim
        if len(q_norm_bytes) != 2 * hd or len(k_norm_bytes) != 2 * hd:
            raise ValueError("q_norm/k_norm must be head_dim bf16 values each")
        self.state.qknorm_params[layer_idx] = gpu.upload_buffer(f"qknorm_params_{layer_idx}",
                                                                bytes(q_norm_bytes) + bytes(k_norm_bytes))

    def _cache(self, layer_idx: int) -> ops.KvCacheView:
        return ops.KvCacheView(self.kv_dtype, self.state.k_cache[layer_idx], self.state.v_cache[layer_idx], 0)

    def fused_split_qknorm_kvstore(self, gpu: GpuContext, layer_idx: int) -> None:
        """model.rs:486-513."""
        c, s = self.config, self.state
        if self.seq_len >= self.max_seq_len:
            raise IndexError("KV cache is full")
        if self._pos_on_device != self.seq_len:      # model.rs:493-496 writes it per layer; once per token is enough
            gpu.write_buffer(s.position, 0, struct.pack("I", self.seq_len))
            self._pos_on_device = self.seq_len
        # the argument list is marshalled once per layer and cache binding: a single-sequence step is a few
        # microseconds of GPU work, and building ctypes structures per call would cost more than that
        key = ("append", layer_idx, s.k_cache[layer_idx].ptr, s.v_cache[layer_idx].ptr,
               s.qknorm_params[layer_idx].ptr if s.qknorm_params[layer_idx] else 0)
        call = self._calls.get(key)
        if call is None:
            rd = c.rotary_dim
            p = AppendParams(c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.rms_norm_eps, c.rope_theta, rd,
                             rd // 2, rd // 2, int(c.mrope_interleaved), 1, 1, F32, F32, 1, 1, 0)
            cs = self._cache(layer_idx).c_struct()
            vp = C.c_void_p
            args = (gpu.handle, C.byref(p), vp(s.q_out.ptr), vp(s.k_out.ptr), vp(s.v_out.ptr), vp(s.q_proj.ptr),
                    vp(s.q_gate.ptr), C.byref(cs), vp(key[4] or None), vp(s.position.ptr), None, None)
            if len(self._calls) >= 4 * max(1, c.num_hidden_layers) + 16:   # cache swaps rebind buffers
                self._calls.clear()
            call = self._calls[key] = (args, (p, cs))
        st = gpu._L.shady_kv_append_rope(*call[0])
        if st:
            gpu._check(st)

    def gqa_attention(self, gpu: GpuContext, layer_idx: int, fuse_gate: bool = False) -> None:
        """model.rs:516-573.  ``fuse_gate`` folds the following ``sigmoid_mul_gate`` into the epilogue."""
        c, s = self.config, self.state
        seq_len = self.seq_len + 1  # include current token (model.rs:521)
        if self._len_on_device != seq_len:
            gpu.write_buffer(s.seq_len_dev, 0, struct.pack("I", seq_len))
            self._len_on_device = seq_len
        key = ("attend", layer_idx, s.k_cache[layer_idx].ptr, s.v_cache[layer_idx].ptr, bool(fuse_gate))
        call = self._calls.get(key)
        if call is None:
            p = DecodeParams(c.head_dim, c.num_key_value_heads, c.num_attention_heads,
                             c.num_attention_heads // c.num_key_value_heads, self.num_attn_splits, 1, F32, F32)
            cs = self._cache(layer_idx).c_struct()
            vp = C.c_void_p
            args = (gpu.handle, C.byref(p), vp(s.q_proj.ptr), C.byref(cs), vp(s.seq_len_dev.ptr),
                    C.cast(self._len_host, C.POINTER(C.c_uint32)), vp(s.attn_output.ptr), None,
                    vp(s.q_gate.ptr if fuse_gate else None), vp(s.attn_partials.ptr), s.partials_bytes)
            if len(self._calls) >= 4 * max(1, c.num_hidden_layers) + 16:   # cache swaps rebind buffers
                self._calls.clear()
            call = self._calls[key] = (args, (p, cs))
        self._len_host[0] = seq_len
        st = gpu._L.shady_attn_decode(*call[0])
        if st:
            gpu._check(st)

    def sigmoid_mul_gate(self, gpu: GpuContext) -> None:
        """model.rs:576-593 (in place; no temp buffer + copy)."""
        c, s = self.config, self.state
        ops.sigmoid_mul(gpu, s.attn_output, s.q_gate, c.num_attention_heads * c.head_dim)

    def attention_step(self, gpu: GpuContext, layer_idx: int) -> None:
        """The three calls of model.rs:723-725 for one self-attention layer."""
        self.fused_split_qknorm_kvstore(gpu, layer_idx)
        self.gqa_attention(gpu, layer_idx)
        self.sigmoid_mul_gate(gpu)

    # -- cache slots (model.rs:973-1029, KV part) -------------------------------------------------
    def alloc_cache_slot(self, gpu: GpuContext) -> CacheSlot:
        c = self.config
        esz = 4 if self.kv_dtype == F32 else 2
        n = self.max_seq_len * c.num_key_value_heads * c.head_dim * esz
        return CacheSlot([gpu.create_storage_buffer(f"slot_k_{i}", n) for i in range(c.num_hidden_layers)],
                         [gpu.create_storage_buffer(f"slot_v_{i}", n) for i in range(c.num_hidden_layers)], 0)

    def swap_cache(self, slot: CacheSlot) -> None:
        s = self.state
        s.k_cache, slot.k_cache = slot.k_cache, s.k_cache
        s.v_cache, slot.v_cache = slot.v_cache, s.v_cache
        self.seq_len, slot.seq_len = slot.seq_len, self.seq_len
