"""Thin functional wrappers over the C ABI ops.  Arguments are device buffers (``gpu.Buffer``,
CUDA tensors or raw addresses); nothing here computes on the host."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import BF16, F8E4M3, F16, F32, AppendParams, DecodeParams, GptqWeight, KvCache, PrefillParams
from .gpu import GpuContext, _addr

_TORCH_DTYPES = None


def dtype_code(t) -> int:
    """SHADY_* code of a torch dtype / numpy dtype / code."""
    global _TORCH_DTYPES
    if isinstance(t, int):
        return t
    if _TORCH_DTYPES is None:
        import torch
        _TORCH_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}
    if t in _TORCH_DTYPES:
        return _TORCH_DTYPES[t]
    return {np.dtype(np.float32): F32, np.dtype(np.float16): F16}[np.dtype(t)]


@dataclass
class KvCacheView:
    """Where the per-sequence K/V rows live: one allocation with a per-sequence stride, or device
    arrays of per-sequence pointers (see ``shady_kv_cache``)."""

    dtype: int
    k_base: object = None
    v_base: object = None
    seq_stride: int = 0          # elements
    k_ptrs: object = None        # device array of device pointers (uint64) [num_seqs]
    v_ptrs: object = None
    page_table: object = None    # paged cache: device u32 [num_seqs][max_pages_per_seq]; k_base / v_base are the pools
    page_rows: int = 0
    max_pages_per_seq: int = 0
    k_scale: float = 0.0         # 8-bit (e4m3) cache: value = stored * scale; 0 means 1
    v_scale: float = 0.0

    def c_struct(self) -> KvCache:
        return KvCache(_addr(self.k_base) or None, _addr(self.v_base) or None, self.seq_stride,
                       _addr(self.k_ptrs) or None, _addr(self.v_ptrs) or None, self.dtype, self.page_rows,
                       _addr(self.page_table) or None, self.max_pages_per_seq, self.k_scale, self.v_scale, 0)


def kv_append_rope(gpu: GpuContext, *, q_proj_full, k_proj, v_proj, q_out, q_gate, cache: KvCacheView, pos_start,
                   num_heads: int, num_kv_heads: int, head_dim: int, rope_theta: float, rotary_dim: int,
                   interleaved: bool = True, eps: float = 1e-6, qk_norm_bf16=None, num_seqs: int = 1,
                   tokens_per_seq: int = 1, in_dtype: int = F32, q_dtype: int = F32, has_gate: bool = True,
                   write_k_back: bool = True, pos_h=None, pos_w=None, s1_limit: int | None = None,
                   s2_limit: int | None = None) -> None:
    p = AppendParams(num_heads, num_kv_heads, head_dim, eps, rope_theta, rotary_dim,
                     rotary_dim // 2 if s1_limit is None else s1_limit,
                     rotary_dim // 2 if s2_limit is None else s2_limit, int(interleaved), num_seqs,
                     tokens_per_seq, in_dtype, q_dtype, int(has_gate), int(write_k_back), 0)
    c = cache.c_struct()
    gpu._check(gpu._L.shady_kv_append_rope(gpu.handle, C.byref(p), _addr(q_proj_full), _addr(k_proj), _addr(v_proj),
                                           _addr(q_out), _addr(q_gate) or None, C.byref(c),
                                           _addr(qk_norm_bf16) or None, _addr(pos_start), _addr(pos_h) or None,
                                           _addr(pos_w) or None))


def decode_workspace_size(*, head_dim: int, num_kv_heads: int, num_q_heads: int, num_splits: int, num_seqs: int) -> int:
    p = DecodeParams(head_dim, num_kv_heads, num_q_heads, num_q_heads // num_kv_heads, num_splits, num_seqs, F32, F32)
    n = C.c_size_t()
    st = _lib.load().shady_decode_workspace_size(C.byref(p), C.byref(n))
    if st != _lib.OK:
        raise _lib.ShadyError(st, "decode_workspace_size")
    return n.value


def decode_workspace_init(gpu: GpuContext, workspace, workspace_bytes: int, *, head_dim: int, num_kv_heads: int,
                          num_q_heads: int, num_splits: int, num_seqs: int) -> None:
    """Zero the arrival counters at the head of a freshly allocated decode workspace (once)."""
    p = DecodeParams(head_dim, num_kv_heads, num_q_heads, num_q_heads // num_kv_heads, num_splits, num_seqs, F32, F32)
    gpu._check(gpu._L.shady_decode_workspace_init(gpu.handle, C.byref(p), _addr(workspace) or None, workspace_bytes))


def _host_lens(seq_lens_host):
    if seq_lens_host is None:
        return None, None
    arr = np.ascontiguousarray(seq_lens_host, dtype=np.uint32)
    return arr, arr.ctypes.data_as(C.POINTER(C.c_uint32))


def attn_decode(gpu: GpuContext, *, q, cache: KvCacheView, seq_lens, out, head_dim: int, num_kv_heads: int,
                num_q_heads: int, num_seqs: int = 1, num_splits: int = 0, seq_lens_host=None, q_dtype: int = F32,
                out_dtype: int = F32, lse=None, gate=None, workspace=None, workspace_bytes: int = 0) -> None:
    p = DecodeParams(head_dim, num_kv_heads, num_q_heads, num_q_heads // num_kv_heads, num_splits, num_seqs, q_dtype,
                     out_dtype)
    c = cache.c_struct()
    keep, hl = _host_lens(seq_lens_host)
    gpu._check(gpu._L.shady_attn_decode(gpu.handle, C.byref(p), _addr(q), C.byref(c), _addr(seq_lens), hl, _addr(out),
                                        _addr(lse) or None, _addr(gate) or None, _addr(workspace) or None,
                                        workspace_bytes))
    del keep


def attn_decode_static(gpu: GpuContext, *, q, cache: KvCacheView, seq_lens, out, head_dim: int, num_kv_heads: int,
                       num_q_heads: int, num_seqs: int = 1, num_splits: int = 0, seq_lens_host=None,
                       q_dtype: int = F32, out_dtype: int = F32, lse=None, gate=None) -> None:
    """``attn_decode`` for callers that cannot supply a workspace: the scratch is a 4 MiB array inside the
    library.  Raises ``ShadyError`` (status 4) when the launch would need more.  Calls must not overlap on
    the GPU, and the first call on a device should come before any stream capture."""
    p = DecodeParams(head_dim, num_kv_heads, num_q_heads, num_q_heads // num_kv_heads, num_splits, num_seqs, q_dtype,
                     out_dtype)
    c = cache.c_struct()
    keep, hl = _host_lens(seq_lens_host)
    gpu._check(gpu._L.shady_attn_decode_static(gpu.handle, C.byref(p), _addr(q), C.byref(c), _addr(seq_lens), hl,
                                               _addr(out), _addr(lse) or None, _addr(gate) or None))
    del keep


def attn_decode_append(gpu: GpuContext, *, q_proj_full, k_proj, v_proj, cache: KvCacheView, seq_lens, out,
                       num_heads: int, num_kv_heads: int, head_dim: int, rope_theta: float, rotary_dim: int,
                       num_seqs: int = 1, eps: float = 1e-6, qk_norm_bf16=None, in_dtype: int = F32,
                       out_dtype: int = F32, has_gate: bool = True, seq_lens_host=None, lse=None, workspace=None,
                       workspace_bytes: int = 0, num_splits: int = 0) -> None:
    """One launch for append + attend (+ gate): ``seq_lens`` count the token being appended."""
    ap = AppendParams(num_heads, num_kv_heads, head_dim, eps, rope_theta, rotary_dim, rotary_dim // 2, rotary_dim // 2,
                      1, num_seqs, 1, in_dtype, in_dtype, int(has_gate), 0, 0)
    p = DecodeParams(head_dim, num_kv_heads, num_heads, num_heads // num_kv_heads, num_splits, num_seqs, in_dtype,
                     out_dtype)
    c = cache.c_struct()
    keep, hl = _host_lens(seq_lens_host)
    gpu._check(gpu._L.shady_attn_decode_append(gpu.handle, C.byref(ap), C.byref(p), _addr(q_proj_full), _addr(k_proj),
                                               _addr(v_proj), _addr(qk_norm_bf16) or None, C.byref(c), _addr(seq_lens),
                                               hl, _addr(out), _addr(lse) or None, _addr(workspace) or None,
                                               workspace_bytes))
    del keep


def attn_decode_shard(gpu: GpuContext, *, q, cache: KvCacheView, seq_lens, records, head_dim: int, num_kv_heads: int,
                      num_q_heads: int, num_seqs: int = 1, num_splits: int = 0, seq_lens_host=None, q_dtype: int = F32,
                      workspace=None, workspace_bytes: int = 0) -> None:
    """Decode over this rank's rows of each sequence; result as records [num_seqs][nh][hd+2] (out, lse, unused)."""
    p = DecodeParams(head_dim, num_kv_heads, num_q_heads, num_q_heads // num_kv_heads, num_splits, num_seqs, q_dtype,
                     F32)
    c = cache.c_struct()
    keep, hl = _host_lens(seq_lens_host)
    gpu._check(gpu._L.shady_attn_decode_shard(gpu.handle, C.byref(p), _addr(q), C.byref(c), _addr(seq_lens), hl,
                                              _addr(records), _addr(workspace) or None, workspace_bytes))
    del keep


def attn_decode_partials(gpu: GpuContext, *, q, cache: KvCacheView, seq_lens, partials, head_dim: int,
                         num_kv_heads: int, num_q_heads: int, num_splits: int, q_dtype: int = F32) -> None:
    p = DecodeParams(head_dim, num_kv_heads, num_q_heads, num_q_heads // num_kv_heads, num_splits, 1, q_dtype, F32)
    c = cache.c_struct()
    gpu._check(gpu._L.shady_attn_decode_partials(gpu.handle, C.byref(p), _addr(q), C.byref(c), _addr(seq_lens),
                                                 _addr(partials)))


def attn_reduce(gpu: GpuContext, *, partials, out, head_dim: int, num_splits: int, num_heads: int,
                split_stride: int | None = None, head_stride: int | None = None, out_dtype: int = F32,
                gate=None) -> None:
    """Defaults to the reference layout [nh][ns][hd+2] (gqa_reduce.wgsl:7-12)."""
    ss = head_dim + 2 if split_stride is None else split_stride
    hs = num_splits * (head_dim + 2) if head_stride is None else head_stride
    gpu._check(gpu._L.shady_attn_reduce(gpu.handle, head_dim, num_splits, num_heads, ss, hs, _addr(partials),
                                        _addr(out), out_dtype, _addr(gate) or None))


def attn_prefill(gpu: GpuContext, *, q, cache: KvCacheView, out, head_dim: int, num_kv_heads: int, num_q_heads: int,
                 num_seqs: int, seq_len: int, dtype: int = BF16) -> None:
    p = PrefillParams(head_dim, num_kv_heads, num_q_heads, num_seqs, seq_len, dtype)
    c = cache.c_struct()
    gpu._check(gpu._L.shady_attn_prefill(gpu.handle, C.byref(p), _addr(q), C.byref(c), _addr(out)))


def prefill_workspace_size(*, head_dim: int, num_kv_heads: int, num_q_heads: int, num_seqs: int, seq_len: int,
                           dtype: int = BF16) -> int:
    p = PrefillParams(head_dim, num_kv_heads, num_q_heads, num_seqs, seq_len, dtype)
    n = C.c_size_t()
    st = _lib.load().shady_prefill_workspace_size(C.byref(p), C.byref(n))
    if st != _lib.OK:
        raise _lib.ShadyError(st, "prefill_workspace_size")
    return n.value


def attn_prefill_append(gpu: GpuContext, *, q_proj_full, k_proj, v_proj, cache: KvCacheView, out, workspace,
                        workspace_bytes: int, num_heads: int, num_kv_heads: int, head_dim: int, num_seqs: int,
                        seq_len: int, rope_theta: float, rotary_dim: int, dtype: int = BF16, eps: float = 1e-6,
                        qk_norm_bf16=None, has_gate: bool = False) -> None:
    """The prefill step from the projections: K/V rows [0, seq_len) of every cache written (K normed + rotated),
    Q normed + rotated inside the attention kernel, causal attention, sigmoid gate."""
    ap = AppendParams(num_heads, num_kv_heads, head_dim, eps, rope_theta, rotary_dim, rotary_dim // 2, rotary_dim // 2,
                      1, num_seqs, seq_len, dtype, dtype, int(has_gate), 0, 0)
    p = PrefillParams(head_dim, num_kv_heads, num_heads, num_seqs, seq_len, dtype)
    c = cache.c_struct()
    gpu._check(gpu._L.shady_attn_prefill_append(gpu.handle, C.byref(ap), C.byref(p), _addr(q_proj_full), _addr(k_proj),
                                                _addr(v_proj), _addr(qk_norm_bf16) or None, C.byref(c), _addr(out),
                                                _addr(workspace), workspace_bytes))


class _ListedBatch:
    """Host arrays of a listed prefill batch, kept alive for the duration of the call."""

    def __init__(self, seq_lens, k_ptrs=None, v_ptrs=None):
        n = len(seq_lens)
        self.lens = (C.c_uint32 * n)(*[int(v) for v in seq_lens])
        self.k = (C.c_void_p * n)(*[int(v) for v in k_ptrs]) if k_ptrs is not None else None
        self.v = (C.c_void_p * n)(*[int(v) for v in v_ptrs]) if v_ptrs is not None else None
        self.c = _lib.PrefillBatch(C.cast(self.lens, C.c_void_p), C.cast(self.k, C.c_void_p) if self.k is not None else None,
                                   C.cast(self.v, C.c_void_p) if self.v is not None else None)


def prefill_ragged_workspace_size(*, seq_lens, head_dim: int, num_kv_heads: int, num_q_heads: int, dtype: int = BF16,
                                  with_append: bool = False) -> int:
    p = PrefillParams(head_dim, num_kv_heads, num_q_heads, len(seq_lens), 0, dtype)
    lens = (C.c_uint32 * len(seq_lens))(*[int(v) for v in seq_lens])
    n = C.c_size_t()
    st = _lib.load().shady_prefill_ragged_workspace_size(C.byref(p), C.cast(lens, C.c_void_p), int(with_append), C.byref(n))
    if st != _lib.OK:
        raise _lib.ShadyError(st, "prefill_ragged_workspace_size")
    return n.value


def attn_prefill_ragged(gpu: GpuContext, *, q, cache: KvCacheView, out, seq_lens, workspace, workspace_bytes: int,
                        head_dim: int, num_kv_heads: int, num_q_heads: int, dtype: int = BF16, k_ptrs=None,
                        v_ptrs=None) -> None:
    """Causal attention of prompts of different lengths; ``q`` and ``out`` packed ``[sum T_i][nh][hd]``.  ``k_ptrs`` /
    ``v_ptrs``: the per-sequence cache addresses as host integers when ``cache`` is a pointer-array cache."""
    p = PrefillParams(head_dim, num_kv_heads, num_q_heads, len(seq_lens), 0, dtype)
    b = _ListedBatch(seq_lens, k_ptrs, v_ptrs)
    c = cache.c_struct()
    gpu._check(gpu._L.shady_attn_prefill_ragged(gpu.handle, C.byref(p), C.byref(b.c), _addr(q), C.byref(c), _addr(out),
                                                _addr(workspace), workspace_bytes))


def attn_prefill_append_ragged(gpu: GpuContext, *, q_proj_full, k_proj, v_proj, cache: KvCacheView, out, seq_lens,
                               workspace, workspace_bytes: int, num_heads: int, num_kv_heads: int, head_dim: int,
                               rope_theta: float, rotary_dim: int, dtype: int = BF16, eps: float = 1e-6,
                               qk_norm_bf16=None, has_gate: bool = False, k_ptrs=None, v_ptrs=None) -> None:
    """The prefill step from the projections for prompts of different lengths (everything packed token-major)."""
    S = len(seq_lens)
    ap = AppendParams(num_heads, num_kv_heads, head_dim, eps, rope_theta, rotary_dim, rotary_dim // 2, rotary_dim // 2,
                      1, S, 0, dtype, dtype, int(has_gate), 0, 0)
    p = PrefillParams(head_dim, num_kv_heads, num_heads, S, 0, dtype)
    b = _ListedBatch(seq_lens, k_ptrs, v_ptrs)
    c = cache.c_struct()
    gpu._check(gpu._L.shady_attn_prefill_append_ragged(gpu.handle, C.byref(ap), C.byref(p), C.byref(b.c),
                                                       _addr(q_proj_full), _addr(k_proj), _addr(v_proj),
                                                       _addr(qk_norm_bf16) or None, C.byref(c), _addr(out),
                                                       _addr(workspace), workspace_bytes))


@dataclass
class GptqMatrix:
    """One symmetric INT4 weight in the reference's layout (src/weights.rs:252-257): ``qweight`` device u32
    [K/8][N], ``scales`` device f16 [K/group_size][N]."""

    qweight: object
    scales: object
    K: int
    N: int
    group_size: int

    def c_struct(self) -> GptqWeight:
        return GptqWeight(_addr(self.qweight), _addr(self.scales), self.K, self.N, self.group_size, 0)


def gptq_matvec(gpu: GpuContext, w: GptqMatrix, x, y, num_vecs: int = 1) -> None:
    """``Model::gptq_matvec`` (model.rs:357-381): y[v] = W^T x[v], f32."""
    c = w.c_struct()
    gpu._check(gpu._L.shady_gptq_matvec(gpu.handle, C.byref(c), _addr(x), _addr(y), num_vecs))


def qkv_proj_append(gpu: GpuContext, *, wq: GptqMatrix, wk: GptqMatrix, wv: GptqMatrix, x, q_out, q_gate,
                    cache: KvCacheView, pos_start, num_heads: int, num_kv_heads: int, head_dim: int, rope_theta: float,
                    rotary_dim: int, interleaved: bool = True, eps: float = 1e-6, qk_norm_bf16=None, num_seqs: int = 1,
                    q_dtype: int = F32, has_gate: bool = True, pos_h=None, pos_w=None) -> None:
    """The q/k/v projections of one token per sequence and the append (model.rs:698-714 + 723) in one launch."""
    p = AppendParams(num_heads, num_kv_heads, head_dim, eps, rope_theta, rotary_dim, rotary_dim // 2, rotary_dim // 2,
                     int(interleaved), num_seqs, 1, F32, q_dtype, int(has_gate), 0, 0)
    cq, ck, cv, c = wq.c_struct(), wk.c_struct(), wv.c_struct(), cache.c_struct()
    gpu._check(gpu._L.shady_qkv_proj_append(gpu.handle, C.byref(p), C.byref(cq), C.byref(ck), C.byref(cv), _addr(x),
                                            _addr(q_out), _addr(q_gate) or None, C.byref(c), _addr(qk_norm_bf16) or None,
                                            _addr(pos_start), _addr(pos_h) or None, _addr(pos_w) or None))


def sigmoid_mul(gpu: GpuContext, x, gate, n: int) -> None:
    gpu._check(gpu._L.shady_sigmoid_mul(gpu.handle, _addr(x), _addr(gate), n))


def fill_randn(gpu: GpuContext, dst, n: int, dtype: int, seed: int, tensor_id: int, first_idx: int = 0) -> None:
    gpu._check(gpu._L.shady_fill_randn(gpu.handle, _addr(dst), n, dtype, seed, tensor_id, first_idx))
