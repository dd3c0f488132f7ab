"""ctypes binding of ``libshady_attn.so`` (the C ABI in ``include/shady_attn.h``).

There is no fallback: if the CUDA library is missing or a call fails, this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# SHADY_ATTN_LIB points at another build of the same library (kernel tuning experiments)
LIB_PATH = os.environ.get("SHADY_ATTN_LIB") or os.path.join(_PKG, "libshady_attn.so")

OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE, ERR_TIMEOUT = range(6)
F32, F16, BF16, F8E4M3, F8E5M2 = 0, 1, 2, 3, 4

# every symbol include/shady_attn.h declares
EXPORTS = [
    "shady_ctx_create", "shady_ctx_destroy", "shady_last_error", "shady_ctx_stream", "shady_ctx_launch_count",
    "shady_ctx_set_wait_limits",
    "shady_buffer_create", "shady_buffer_free", "shady_buffer_write", "shady_buffer_read", "shady_buffer_copy",
    "shady_host_device_ptr",
    "shady_flush", "shady_synchronize", "shady_kv_append_rope", "shady_decode_workspace_size", "shady_decode_workspace_init",
    "shady_attn_decode", "shady_attn_decode_static", "shady_attn_decode_shard", "shady_attn_decode_append", "shady_attn_decode_partials", "shady_attn_reduce", "shady_attn_prefill",
    "shady_prefill_workspace_size", "shady_attn_prefill_append",
    "shady_prefill_ragged_workspace_size", "shady_attn_prefill_ragged", "shady_attn_prefill_append_ragged",
    "shady_gptq_matvec", "shady_qkv_proj_append",
    "shady_sigmoid_mul", "shady_fill_randn", "shady_ipc_export", "shady_ipc_open", "shady_ipc_close",
    "shady_combine_p2p_buffer_size", "shady_attn_combine_p2p", "shady_attn_decode_shard_p2p",
]


class ShadyError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"shady_attn status {code}: {msg}")
        self.code = code


class KvCache(C.Structure):
    _fields_ = [("d_k_base", C.c_void_p), ("d_v_base", C.c_void_p), ("seq_stride", C.c_uint64),
                ("d_k_ptrs", C.c_void_p), ("d_v_ptrs", C.c_void_p), ("dtype", C.c_uint32),
                ("page_rows", C.c_uint32), ("d_page_table", C.c_void_p), ("max_pages_per_seq", C.c_uint32),
                ("k_scale", C.c_float), ("v_scale", C.c_float), ("_pad", C.c_uint32)]


class AppendParams(C.Structure):
    _fields_ = [("num_heads", C.c_uint32), ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("eps", C.c_float), ("rope_theta", C.c_float), ("rotary_dim", C.c_uint32),
                ("s1_limit", C.c_uint32), ("s2_limit", C.c_uint32), ("interleaved", C.c_uint32),
                ("num_seqs", C.c_uint32), ("tokens_per_seq", C.c_uint32), ("in_dtype", C.c_uint32),
                ("q_dtype", C.c_uint32), ("has_gate", C.c_uint32), ("write_k_back", C.c_uint32),
                ("_pad", C.c_uint32)]


class DecodeParams(C.Structure):
    _fields_ = [("head_dim", C.c_uint32), ("num_kv_heads", C.c_uint32), ("num_q_heads", C.c_uint32),
                ("heads_per_kv", C.c_uint32), ("num_splits", C.c_uint32), ("num_seqs", C.c_uint32),
                ("q_dtype", C.c_uint32), ("out_dtype", C.c_uint32)]


class GptqWeight(C.Structure):
    _fields_ = [("d_qweight", C.c_void_p), ("d_scales", C.c_void_p), ("K", C.c_uint32), ("N", C.c_uint32),
                ("group_size", C.c_uint32), ("_pad", C.c_uint32)]


class PrefillParams(C.Structure):
    _fields_ = [("head_dim", C.c_uint32), ("num_kv_heads", C.c_uint32), ("num_q_heads", C.c_uint32),
                ("num_seqs", C.c_uint32), ("seq_len", C.c_uint32), ("dtype", C.c_uint32)]


class PrefillBatch(C.Structure):
    _fields_ = [("h_seq_lens", C.c_void_p), ("h_k_ptrs", C.c_void_p), ("h_v_ptrs", C.c_void_p)]


_lib = None


def load() -> C.CDLL:
    """Load the shared library and declare the prototypes.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: run `python -m shady_thinker_b200.build` "
                          "(there is no CPU or PyTorch fallback for this path)")
    L = C.CDLL(LIB_PATH)
    vp, u32p, f32p, sz = C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t
    L.shady_ctx_create.argtypes = [C.c_int, vp, C.POINTER(vp)]
    L.shady_ctx_destroy.argtypes = [vp]
    L.shady_last_error.argtypes = [vp]
    L.shady_last_error.restype = C.c_char_p
    L.shady_ctx_stream.argtypes = [vp]
    L.shady_ctx_stream.restype = vp
    L.shady_ctx_launch_count.argtypes = [vp]
    L.shady_ctx_launch_count.restype = C.c_uint64
    L.shady_ctx_set_wait_limits.argtypes = [vp, C.c_uint32, C.c_uint32, C.c_uint32]
    L.shady_buffer_create.argtypes = [vp, sz, C.POINTER(vp)]
    L.shady_buffer_free.argtypes = [vp, vp]
    L.shady_buffer_write.argtypes = [vp, vp, sz, vp, sz]
    L.shady_buffer_read.argtypes = [vp, vp, sz, vp, sz]
    L.shady_buffer_copy.argtypes = [vp, vp, vp, sz]
    L.shady_host_device_ptr.argtypes = [vp, vp, C.POINTER(vp)]
    L.shady_flush.argtypes = [vp]
    L.shady_synchronize.argtypes = [vp]
    L.shady_kv_append_rope.argtypes = [vp, C.POINTER(AppendParams), vp, vp, vp, vp, f32p, C.POINTER(KvCache), vp,
                                       u32p, u32p, u32p]
    L.shady_decode_workspace_size.argtypes = [C.POINTER(DecodeParams), C.POINTER(sz)]
    L.shady_decode_workspace_init.argtypes = [vp, C.POINTER(DecodeParams), vp, sz]
    L.shady_attn_decode.argtypes = [vp, C.POINTER(DecodeParams), vp, C.POINTER(KvCache), u32p,
                                    C.POINTER(C.c_uint32), vp, f32p, f32p, vp, sz]
    L.shady_attn_decode_static.argtypes = [vp, C.POINTER(DecodeParams), vp, C.POINTER(KvCache), u32p,
                                           C.POINTER(C.c_uint32), vp, f32p, f32p]
    L.shady_attn_decode_append.argtypes = [vp, C.POINTER(AppendParams), C.POINTER(DecodeParams), vp, vp, vp, vp,
                                           C.POINTER(KvCache), u32p, C.POINTER(C.c_uint32), vp, f32p, vp, sz]
    L.shady_attn_decode_shard.argtypes = [vp, C.POINTER(DecodeParams), vp, C.POINTER(KvCache), u32p,
                                          C.POINTER(C.c_uint32), f32p, vp, sz]
    L.shady_attn_decode_partials.argtypes = [vp, C.POINTER(DecodeParams), vp, C.POINTER(KvCache), u32p, f32p]
    L.shady_attn_reduce.argtypes = [vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint64, f32p, vp,
                                    C.c_uint32, f32p]
    L.shady_attn_prefill.argtypes = [vp, C.POINTER(PrefillParams), vp, C.POINTER(KvCache), vp]
    L.shady_prefill_workspace_size.argtypes = [C.POINTER(PrefillParams), C.POINTER(sz)]
    L.shady_attn_prefill_append.argtypes = [vp, C.POINTER(AppendParams), C.POINTER(PrefillParams), vp, vp, vp, vp,
                                            C.POINTER(KvCache), vp, vp, sz]
    L.shady_prefill_ragged_workspace_size.argtypes = [C.POINTER(PrefillParams), vp, C.c_int, C.POINTER(sz)]
    L.shady_attn_prefill_ragged.argtypes = [vp, C.POINTER(PrefillParams), C.POINTER(PrefillBatch), vp, C.POINTER(KvCache),
                                            vp, vp, sz]
    L.shady_attn_prefill_append_ragged.argtypes = [vp, C.POINTER(AppendParams), C.POINTER(PrefillParams),
                                                   C.POINTER(PrefillBatch), vp, vp, vp, vp, C.POINTER(KvCache), vp, vp, sz]
    L.shady_ipc_export.argtypes = [vp, vp, C.c_char_p]
    L.shady_ipc_open.argtypes = [vp, C.c_char_p, C.POINTER(vp)]
    L.shady_ipc_close.argtypes = [vp, vp]
    L.shady_combine_p2p_buffer_size.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(sz)]
    L.shady_attn_combine_p2p.argtypes = [vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, vp, f32p, vp,
                                         C.c_uint32, f32p]
    L.shady_attn_decode_shard_p2p.argtypes = [vp, C.POINTER(DecodeParams), vp, C.POINTER(KvCache), u32p,
                                              C.POINTER(C.c_uint32), C.c_uint32, C.c_uint32, C.c_uint32, vp, f32p, vp,
                                              C.c_uint32, f32p, vp, sz]
    L.shady_gptq_matvec.argtypes = [vp, C.POINTER(GptqWeight), f32p, f32p, C.c_uint32]
    L.shady_qkv_proj_append.argtypes = [vp, C.POINTER(AppendParams), C.POINTER(GptqWeight), C.POINTER(GptqWeight),
                                        C.POINTER(GptqWeight), f32p, vp, f32p, C.POINTER(KvCache), vp, u32p, u32p, u32p]
    L.shady_sigmoid_mul.argtypes = [vp, f32p, f32p, C.c_uint32]
    L.shady_fill_randn.argtypes = [vp, vp, C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint64, C.c_uint64]
    for name in EXPORTS:
        fn = getattr(L, name)
        if name not in ("shady_last_error", "shady_ctx_stream", "shady_ctx_launch_count"):
            fn.restype = C.c_int
    _lib = L
    return L


def check(ctx_handle, status: int) -> None:
    """Turn a non-zero status into an exception carrying the library's message (the reference
    panics in the same places: gpu.rs:43,68,271)."""
    if status != OK:
        msg = load().shady_last_error(ctx_handle)
        raise ShadyError(status, msg.decode() if msg else "")
