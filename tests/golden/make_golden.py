"""Regenerates ``golden_v1.npz`` from the CPU oracle.

The reference holds no golden vectors for the attention path and its WGSL cannot run here,
so these fixtures pin the ORACLE (a restatement of the shaders), not the reference itself:
they freeze today's oracle outputs so that later edits of the oracle or of the generator
cannot drift silently.  Inputs are not stored — they are a pure function of
(seed, tensor_id, index) through ``oracle.randn`` — only outputs are.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

SEED = 0x5EED

# name -> (nh, nkv, hd, L, num_splits)
DECODE_CASES = {
    "cfg1_f32": (16, 2, 128, 512, 1),          # BASELINE config 1
    "cfg1_f32_split4": (16, 2, 128, 512, 4),
    "hd256_g8": (16, 2, 256, 333, 1),
    "hd64_g1": (4, 4, 64, 37, 3),
}
# name -> (nh, nkv, hd, theta, rotary_dim, interleaved, norm, position)
APPEND_CASES = {
    "cfg1_rope_full": (16, 2, 128, 1e6, 128, True, False, 511),
    "ref_default": (16, 2, 128, 1e7, 32, True, True, 1234),
    "rotate_half_hd256": (16, 2, 256, 1e6, 64, False, True, 131071),
}


def decode_inputs(name, nh, nkv, hd, L):
    tid = sum(map(ord, name))  # stable across runs
    q = O.randn((nh, hd), SEED, 100 + tid)
    k = O.randn((L, nkv, hd), SEED, 200 + tid)
    v = O.randn((L, nkv, hd), SEED, 300 + tid)
    return q, k, v


def append_inputs(name, nh, nkv, hd):
    tid = sum(map(ord, name))
    qf = O.randn((nh, 2, hd), SEED, 400 + tid)
    kp = O.randn((nkv, hd), SEED, 500 + tid)
    vp = O.randn((nkv, hd), SEED, 600 + tid)
    w = O.bf16_bits(O.randn((2 * hd,), SEED, 700 + tid) * np.float32(0.02))
    return qf, kp, vp, w


def run_decode(name):
    nh, nkv, hd, L, ns = DECODE_CASES[name]
    q, k, v = decode_inputs(name, nh, nkv, hd, L)
    out = O.gqa_attention_head(q, k, v, L, num_splits=ns)
    return out if ns == 1 else (out, O.gqa_reduce(out))


def run_append(name):
    nh, nkv, hd, theta, rd, inter, norm, pos = APPEND_CASES[name]
    qf, kp, vp, w = append_inputs(name, nh, nkv, hd)
    kc = np.zeros((pos + 1, nkv, hd), np.float32)
    vc = np.zeros_like(kc)
    q, g, k = O.fused_split_qknorm_kvstore(qf, kp, vp, kc, vc, pos, rope_theta=theta, rotary_dim=rd,
                                           interleaved=inter, qk_norm_bf16=w if norm else None)
    return q, g, k, kc[pos].copy(), vc[pos].copy()


def main():
    out = {}
    for name in DECODE_CASES:
        r = run_decode(name)
        if isinstance(r, tuple):
            out[f"decode/{name}/partials"], out[f"decode/{name}/out"] = r
        else:
            out[f"decode/{name}/out"] = r
    for name in APPEND_CASES:
        for key, arr in zip(("q", "gate", "k", "k_row", "v_row"), run_append(name)):
            out[f"append/{name}/{key}"] = arr
    out["randn/first16"] = O.randn((16,), SEED, 1)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_v1.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
