"""ctypes front end of the CPU oracle (``shady_oracle.c``).

TEST INFRASTRUCTURE ONLY: importable from ``tests/``, from the smoke check and from the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark.  The product package never
imports this module.  Parity is unpinned by the reference (it holds no golden vectors for
this path); see the header of ``shady_oracle.c``.

Every wrapper names the reference shader it restates:
  gqa_attention_head   src/shaders/gqa_attention_head.wgsl:30-124
  gqa_reduce           src/shaders/gqa_reduce.wgsl:20-65
  fused_split_qknorm_kvstore  src/shaders/fused_split_qknorm_kvstore.wgsl:106-230
  sigmoid_mul          src/shaders/sigmoid_mul.wgsl:16-23
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libshady_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc, no GPU needed)."""
    src = os.path.join(_HERE, "shady_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "libshady_oracle.so"])
    return _SO


class QkNormParams(C.Structure):
    """Header of the qknorm uniform (fused_split_qknorm_kvstore.wgsl:12-21) plus the
    constants model.rs:32-54 injects into the shader source."""

    _fields_ = [
        ("num_heads", C.c_uint32),
        ("num_kv_heads", C.c_uint32),
        ("head_dim", C.c_uint32),
        ("eps", C.c_float),
        ("cache_position", C.c_uint32),
        ("position", C.c_uint32),
        ("position_h", C.c_uint32),
        ("position_w", C.c_uint32),
        ("rope_theta", C.c_float),
        ("partial_dim", C.c_uint32),
        ("s1_limit", C.c_uint32),
        ("s2_limit", C.c_uint32),
        ("interleaved", C.c_uint32),
        ("has_norm", C.c_uint32),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        f32p, f64p, u16p, u32p = (C.POINTER(C.c_float), C.POINTER(C.c_double), C.POINTER(C.c_uint16),
                                  C.POINTER(C.c_uint32))
        L.oracle_num_threads.restype = C.c_int
        L.oracle_gqa_attention_head_f32.argtypes = [f32p, f32p, f32p, f32p] + [C.c_uint32] * 6 + [C.c_int]
        L.oracle_gqa_reduce_f32.argtypes = [f32p, f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int]
        L.oracle_fused_split_qknorm_kvstore_f32.argtypes = [C.POINTER(QkNormParams), f32p, f32p, f32p, f32p,
                                                            f32p, f32p, f32p, u16p]
        L.oracle_sigmoid_mul_f32.argtypes = [f32p, f32p, f32p, C.c_uint32]
        L.oracle_gptq_matvec_f32.argtypes = [f32p, u32p, u32p, f32p, C.c_uint32, C.c_uint32, C.c_uint32]
        L.oracle_attention_f64.argtypes = [f32p, f32p, f32p, f64p] + [C.c_uint32] * 5 + [C.c_int]
        L.oracle_causal_prefill_f32.argtypes = [f32p, f32p, f32p, f32p] + [C.c_uint32] * 5 + [C.c_int]
        L.oracle_causal_prefill_f64.argtypes = [f32p, f32p, f32p, f64p] + [C.c_uint32] * 5 + [C.c_int]
        L.oracle_batched_decode_f32.argtypes = [f32p, C.POINTER(f32p), C.POINTER(f32p), u32p, C.c_uint32, f32p,
                                                C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int]
        L.oracle_randn_at.argtypes = [C.c_uint64] * 3
        L.oracle_randn_at.restype = C.c_float
        L.oracle_fill_randn.argtypes = [f32p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64]
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray, ty=C.c_float):
    return a.ctypes.data_as(C.POINTER(ty))


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def gqa_attention_head(q, k_cache, v_cache, seq_len: int, num_splits: int = 1, threads: int = 1) -> np.ndarray:
    """q [nh,hd]; k_cache/v_cache [>=seq_len, nkv, hd].  Returns [nh,hd] (num_splits==1) or the
    partials buffer [nh, num_splits, hd+2]."""
    q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
    nh, hd = q.shape
    nkv = k_cache.shape[1]
    assert hd <= 256 and nh % nkv == 0 and k_cache.shape[0] >= seq_len
    out = np.empty((nh, hd) if num_splits == 1 else (nh, num_splits, hd + 2), np.float32)
    lib().oracle_gqa_attention_head_f32(_p(q), _p(k_cache), _p(v_cache), _p(out), seq_len, hd, nkv, nh,
                                        nh // nkv, num_splits, threads)
    return out


def gqa_reduce(partials, skip_empty: bool = False) -> np.ndarray:
    partials = _f32(partials)
    nh, ns, hd2 = partials.shape
    out = np.empty((nh, hd2 - 2), np.float32)
    lib().oracle_gqa_reduce_f32(_p(partials), _p(out), hd2 - 2, ns, nh, int(skip_empty))
    return out


def rotary_dim(head_dim: int, partial_rotary_factor: float) -> int:
    """model.rs:33: ``(config.head_dim as f32 * config.partial_rotary_factor) as u32``"""
    return int(np.float32(head_dim) * np.float32(partial_rotary_factor))


def fused_split_qknorm_kvstore(q_proj_full, k_proj, v_proj, k_cache, v_cache, position: int, *,
                               rope_theta: float, rotary_dim: int, interleaved: bool = True, eps: float = 1e-6,
                               qk_norm_bf16=None, cache_position=None):
    """One token.  q_proj_full [nh,2,hd]; k_proj,v_proj [nkv,hd]; caches [max,nkv,hd] f32 (written in
    place at ``cache_position``).  Returns (q_proj [nh,hd], q_gate [nh,hd], k_out [nkv,hd])."""
    q_proj_full = _f32(q_proj_full)
    nh, two, hd = q_proj_full.shape
    assert two == 2 and hd <= 256
    k = _f32(k_proj).copy()
    v = _f32(v_proj)
    nkv = k.shape[0]
    assert k_cache.dtype == np.float32 and k_cache.flags.c_contiguous
    assert v_cache.dtype == np.float32 and v_cache.flags.c_contiguous
    p = QkNormParams(nh, nkv, hd, eps, position if cache_position is None else cache_position, position,
                     position, position, rope_theta, rotary_dim, rotary_dim // 2, rotary_dim // 2,
                     int(interleaved), int(qk_norm_bf16 is not None))
    w = None
    if qk_norm_bf16 is not None:
        w = np.ascontiguousarray(qk_norm_bf16, dtype=np.uint16)
        assert w.size == 2 * hd
    q_out = np.empty((nh, hd), np.float32)
    g_out = np.empty((nh, hd), np.float32)
    lib().oracle_fused_split_qknorm_kvstore_f32(C.byref(p), _p(q_proj_full), _p(k), _p(v), _p(q_out), _p(g_out),
                                                _p(k_cache), _p(v_cache),
                                                _p(w, C.c_uint16) if w is not None else None)
    return q_out, g_out, k


def sigmoid_mul(x, gate) -> np.ndarray:
    x, gate = _f32(x).ravel(), _f32(gate).ravel()
    out = np.empty_like(x)
    lib().oracle_sigmoid_mul_f32(_p(x), _p(gate), _p(out), x.size)
    return out


def gptq_matvec(x, qweight, scales_f16, group_size: int) -> np.ndarray:
    """x [K] f32; qweight [K/8, N] uint32; scales_f16 [K/group_size, N] float16 (packed two per u32 for the C side, as
    the shader reads them).  Returns [N] f32 (gptq_matvec.wgsl)."""
    x = _f32(x)
    qw = np.ascontiguousarray(qweight, dtype=np.uint32)
    sc = np.ascontiguousarray(scales_f16, dtype=np.float16)
    K, N = x.size, qw.shape[1]
    assert qw.shape[0] * 8 == K and sc.shape == (K // group_size, N) and (sc.size % 2) == 0
    out = np.empty(N, np.float32)
    lib().oracle_gptq_matvec_f32(_p(x), _p(qw, C.c_uint32), _p(sc.view(np.uint32), C.c_uint32), _p(out), K, N, group_size)
    return out


def attention_f64(q, k_cache, v_cache, seq_len: int, threads: int = 1) -> np.ndarray:
    q, k_cache, v_cache = _f32(q), _f32(k_cache), _f32(v_cache)
    nh, hd = q.shape
    nkv = k_cache.shape[1]
    out = np.empty((nh, hd), np.float64)
    lib().oracle_attention_f64(_p(q), _p(k_cache), _p(v_cache), _p(out, C.c_double), seq_len, hd, nkv, nh,
                               nh // nkv, threads)
    return out


def causal_prefill(q, k, v, f64: bool = False, threads: int = 0) -> np.ndarray:
    """q [T,nh,hd], k/v [T,nkv,hd] already normed/roped; the token loop of inference.rs:93-95."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    T, nh, hd = q.shape
    nkv = k.shape[1]
    threads = threads or num_threads()
    if f64:
        out = np.empty((T, nh, hd), np.float64)
        lib().oracle_causal_prefill_f64(_p(q), _p(k), _p(v), _p(out, C.c_double), T, hd, nkv, nh, nh // nkv,
                                        threads)
    else:
        out = np.empty((T, nh, hd), np.float32)
        lib().oracle_causal_prefill_f32(_p(q), _p(k), _p(v), _p(out), T, hd, nkv, nh, nh // nkv, threads)
    return out


def batched_decode(q, k_list, v_list, seq_lens, threads: int = 0) -> np.ndarray:
    """q [S,nh,hd]; k_list[i]/v_list[i] [>=L_i,nkv,hd] f32.  Sequence-parallel over ``threads``."""
    q = _f32(q)
    S, nh, hd = q.shape
    ks = [_f32(k) for k in k_list]
    vs = [_f32(v) for v in v_list]
    nkv = ks[0].shape[1]
    f32p = C.POINTER(C.c_float)
    kp = (f32p * S)(*[_p(k) for k in ks])
    vp = (f32p * S)(*[_p(v) for v in vs])
    lens = np.ascontiguousarray(seq_lens, dtype=np.uint32)
    out = np.empty((S, nh, hd), np.float32)
    lib().oracle_batched_decode_f32(_p(q), kp, vp, _p(lens, C.c_uint32), S, _p(out), hd, nkv, nh, nh // nkv,
                                    threads or num_threads())
    return out


def randn(shape, seed: int, tensor_id: int, first_idx: int = 0) -> np.ndarray:
    """Counter-based N(0,1): element i is a pure function of (seed, tensor_id, first_idx+i)."""
    out = np.empty(shape, np.float32)
    lib().oracle_fill_randn(_p(out), out.size, seed, tensor_id, first_idx)
    return out


# ---- storage-dtype rounding helpers (RNE), so 16-bit tests feed the oracle what the GPU sees ----

def round_bf16(a) -> np.ndarray:
    u = _f32(a).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def bf16_bits(a) -> np.ndarray:
    return (round_bf16(a).view(np.uint32) >> 16).astype(np.uint16)


def round_f16(a) -> np.ndarray:
    return _f32(a).astype(np.float16).astype(np.float32)


def _f8_stored(a, scale: float, man_bits: int, min_exp: int, max_val: float) -> np.ndarray:
    """``a * (1/scale)`` in f32 (what the append kernels compute), rounded to nearest even onto the grid of an 8-bit
    float with ``man_bits`` mantissa bits whose smallest normal number is 2^min_exp (subnormals below it), saturated
    at +-max_val.  Returned as f32 values on that grid."""
    x = _f32(a) * (np.float32(1.0) / np.float32(scale)) if scale != 1.0 else _f32(a)
    ax = np.minimum(np.abs(x.astype(np.float64)), max_val)
    e = np.floor(np.log2(np.maximum(ax, 2.0 ** -40)))
    e = np.maximum(e, float(min_exp))             # below the smallest normal the grid is the subnormal one
    step = 2.0 ** (e - man_bits)
    q = np.minimum(np.rint(ax / step) * step, max_val)   # numpy rounds halves to even
    return (np.sign(x) * q).astype(np.float32).reshape(np.shape(a))


def e4m3_stored(a, scale: float = 1.0) -> np.ndarray:
    """The e4m3 values (as f32) an 8-bit cache stores for ``a``: 3 mantissa bits, subnormal step 2^-9, +-448."""
    return _f8_stored(a, scale, 3, -6, 448.0)


def e5m2_stored(a, scale: float = 1.0) -> np.ndarray:
    """The e5m2 values (as f32) an 8-bit cache stores for ``a``: 2 mantissa bits, subnormal step 2^-16, +-57344."""
    return _f8_stored(a, scale, 2, -14, 57344.0)


def round_e4m3(a, scale: float = 1.0) -> np.ndarray:
    """What an 8-bit e4m3 cache with this scale holds for ``a``, dequantised: stored value times scale, as f32."""
    return (e4m3_stored(a, scale).astype(np.float64) * np.float64(np.float32(scale))).astype(np.float32)


def round_e5m2(a, scale: float = 1.0) -> np.ndarray:
    return (e5m2_stored(a, scale).astype(np.float64) * np.float64(np.float32(scale))).astype(np.float32)
