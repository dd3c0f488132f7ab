"""The C++ host mirror (include/shady_host.hpp): it compiles and links against the C ABI library on CPU, and on a
GPU a compiled driver runs the reference's token loop through it and matches the oracle."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "host_driver.cpp")


def _build(tmp_path):
    from shady_thinker_b200 import build
    build.build()
    exe = str(tmp_path / "host_driver")
    pkg = os.path.join(ROOT, "shady_thinker_b200")
    cmd = ["/usr/bin/g++", "-std=c++17", "-O2", "-I", os.path.join(ROOT, "include"), SRC, "-o", exe, "-L", pkg,
           "-l:libshady_attn.so", f"-Wl,-rpath,{pkg}", "-Wl,--allow-shlib-undefined"]
    subprocess.check_call(cmd)
    return exe


def test_host_mirror_compiles_and_links(tmp_path):
    exe = _build(tmp_path)
    assert os.path.exists(exe)


@pytest.mark.gpu
def test_cpp_token_loop_matches_oracle(tmp_path, oracle):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    exe = _build(tmp_path)
    nh, nkv, hd, T, layers, theta, prf = 16, 2, 128, 12, 2, 1e6, 0.25
    rd = int(np.float32(hd) * np.float32(prf))
    w = [oracle.bf16_bits(oracle.randn((2 * hd,), 21, 90 + l) * np.float32(0.02)) for l in range(layers)]
    inp = tmp_path / "in.bin"
    with open(inp, "wb") as f:
        np.array([nh, nkv, hd, T, layers], np.uint32).tofile(f)
        np.array([theta, prf], np.float32).tofile(f)
        for l in range(layers):
            w[l].tofile(f)
        toks = []
        for t in range(T):
            for l in range(layers):
                qf = oracle.randn((nh, 2, hd), 21, 1000 + 10 * t + l)
                kp = oracle.randn((nkv, hd), 21, 2000 + 10 * t + l)
                vp = oracle.randn((nkv, hd), 21, 3000 + 10 * t + l)
                qf.tofile(f); kp.tofile(f); vp.tofile(f)
                toks.append((qf, kp, vp))
    outp = tmp_path / "out.bin"
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = os.path.dirname(torch.__file__) + "/lib:" + env.get("LD_LIBRARY_PATH", "")
    r = subprocess.run([exe, str(inp), str(outp)], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0, r.stderr
    got = np.fromfile(outp, np.float32).reshape(T, layers, nh, hd)
    okc = [np.zeros((T + 1, nkv, hd), np.float32) for _ in range(layers)]
    ovc = [np.zeros((T + 1, nkv, hd), np.float32) for _ in range(layers)]
    i = 0
    for t in range(T):
        for l in range(layers):
            qf, kp, vp = toks[i]; i += 1
            oq, og, _ = oracle.fused_split_qknorm_kvstore(qf, kp, vp, okc[l], ovc[l], t, rope_theta=theta, rotary_dim=rd,
                                                          qk_norm_bf16=w[l])
            want = oracle.sigmoid_mul(oracle.gqa_attention_head(oq, okc[l], ovc[l], t + 1), og).reshape(nh, hd)
            assert np.abs(got[t, l] - want).max() <= 1e-3, (t, l)
