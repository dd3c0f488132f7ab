"""GPU parity of the KV append (a-3: Q/gate split + RMSNorm + (m)RoPE + cache store) against the oracle."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from _util import ATOL_F32, TORCH_DT, rounded, to_dev, to_host
from shady_thinker_b200 import ops
from shady_thinker_b200._lib import BF16, F16, F32

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _golden_module():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def _append_one(gpu, qf, kp, vp, pos, *, theta, rd, inter, w, kv_dt=F32, rows=None):
    nh, _, hd = qf.shape
    nkv = kp.shape[0]
    rows = rows or pos + 1
    d_kc = torch.zeros((rows, nkv, hd), dtype=TORCH_DT[kv_dt], device="cuda")
    d_vc = torch.zeros_like(d_kc)
    d_k = to_dev(kp)
    d_q = torch.empty((nh, hd), device="cuda")
    d_g = torch.empty((nh, hd), device="cuda")
    d_w = torch.from_numpy(w.view(np.int16)).cuda() if w is not None else None
    d_pos = torch.tensor([pos], dtype=torch.int32).cuda()
    ops.kv_append_rope(gpu, q_proj_full=to_dev(qf), k_proj=d_k, v_proj=to_dev(vp), q_out=d_q, q_gate=d_g,
                       cache=ops.KvCacheView(kv_dt, d_kc, d_vc, 0), pos_start=d_pos, num_heads=nh, num_kv_heads=nkv,
                       head_dim=hd, rope_theta=theta, rotary_dim=rd, interleaved=inter, qk_norm_bf16=d_w)
    gpu.synchronize()
    return to_host(d_q), to_host(d_g), to_host(d_k), to_host(d_kc), to_host(d_vc)


@pytest.mark.parametrize("name", ["cfg1_rope_full", "ref_default", "rotate_half_hd256"])
def test_golden_cases_f32(gpu_ctx, oracle, name):
    g = _golden_module()
    nh, nkv, hd, theta, rd, inter, norm, pos = g.APPEND_CASES[name]
    qf, kp, vp, w = g.append_inputs(name, nh, nkv, hd)
    q, gate, k, kc, vc = _append_one(gpu_ctx, qf, kp, vp, pos, theta=theta, rd=rd, inter=inter, w=w if norm else None)
    gold = np.load(os.path.join(HERE, "golden", "golden_v1.npz"))
    # pos 131071 * freq is rounded to f32 before cos/sin on both sides: a few 1e-6 is all that is left
    assert np.abs(q - gold[f"append/{name}/q"]).max() <= 2e-5
    assert np.abs(k - gold[f"append/{name}/k"]).max() <= 2e-5
    np.testing.assert_array_equal(gate, gold[f"append/{name}/gate"])
    np.testing.assert_array_equal(kc[pos], k)
    np.testing.assert_array_equal(vc[pos], gold[f"append/{name}/v_row"])
    assert not kc[:pos].any() and not vc[:pos].any()   # only row `pos` is written
    assert max(np.abs(q - gold[f"append/{name}/q"]).max(), np.abs(k - gold[f"append/{name}/k"]).max()) <= ATOL_F32


@pytest.mark.parametrize("kv_dt", [F16, BF16])
def test_cache_rows_are_rne_rounded_oracle_rows(gpu_ctx, oracle, kv_dt):
    nh, nkv, hd, pos = 8, 2, 128, 77
    qf, kp, vp = oracle.randn((nh, 2, hd), 5, 1), oracle.randn((nkv, hd), 5, 2), oracle.randn((nkv, hd), 5, 3)
    w = oracle.bf16_bits(oracle.randn((2 * hd,), 5, 4) * np.float32(0.02))
    _, _, k, kc, vc = _append_one(gpu_ctx, qf, kp, vp, pos, theta=1e6, rd=64, inter=True, w=w, kv_dt=kv_dt)
    okc, ovc = np.zeros((pos + 1, nkv, hd), np.float32), np.zeros((pos + 1, nkv, hd), np.float32)
    oracle.fused_split_qknorm_kvstore(qf, kp, vp, okc, ovc, pos, rope_theta=1e6, rotary_dim=64, qk_norm_bf16=w)
    np.testing.assert_array_equal(vc[pos], rounded(oracle, ovc[pos], kv_dt))     # V is a pure copy: bit-exact
    np.testing.assert_array_equal(kc[pos], rounded(oracle, k, kv_dt))            # K row = RNE(device f32 K)
    ulp = 2.0 ** -10 if kv_dt == F16 else 2.0 ** -7
    assert np.abs(kc[pos] - rounded(oracle, okc[pos], kv_dt)).max() <= ulp * np.abs(okc[pos]).max()


def test_batched_prefill_append_equals_token_loop(gpu_ctx, oracle):
    """tokens_per_seq = T over 2 sequences with different start positions == T single-token oracle calls."""
    S, T, nh, nkv, hd, rd = 2, 9, 4, 2, 128, 32
    starts = [0, 100]
    qf = oracle.randn((S, T, nh, 2, hd), 15, 1)
    kp = oracle.randn((S, T, nkv, hd), 15, 2)
    vp = oracle.randn((S, T, nkv, hd), 15, 3)
    w = oracle.bf16_bits(oracle.randn((2 * hd,), 15, 4) * np.float32(0.02))
    rows = 128
    d_kc = torch.zeros((S, rows, nkv, hd), device="cuda")
    d_vc = torch.zeros_like(d_kc)
    d_q = torch.empty((S, T, nh, hd), device="cuda")
    d_g = torch.empty((S, T, nh, hd), device="cuda")
    d_k = to_dev(kp)
    ops.kv_append_rope(gpu_ctx, q_proj_full=to_dev(qf), k_proj=d_k, v_proj=to_dev(vp), q_out=d_q, q_gate=d_g,
                       cache=ops.KvCacheView(F32, d_kc, d_vc, rows * nkv * hd),
                       pos_start=torch.tensor(starts, dtype=torch.int32).cuda(), num_heads=nh, num_kv_heads=nkv,
                       head_dim=hd, rope_theta=1e7, rotary_dim=rd, qk_norm_bf16=torch.from_numpy(w.view(np.int16)).cuda(),
                       num_seqs=S, tokens_per_seq=T)
    gpu_ctx.synchronize()
    q, kc, vc = to_host(d_q), to_host(d_kc), to_host(d_vc)
    for s in range(S):
        okc, ovc = np.zeros((rows, nkv, hd), np.float32), np.zeros((rows, nkv, hd), np.float32)
        for j in range(T):
            oq, og, _ = oracle.fused_split_qknorm_kvstore(qf[s, j], kp[s, j], vp[s, j], okc, ovc, starts[s] + j,
                                                          rope_theta=1e7, rotary_dim=rd, qk_norm_bf16=w)
            assert np.abs(q[s, j] - oq).max() <= 2e-5
        assert np.abs(kc[s] - okc).max() <= 2e-5
        np.testing.assert_array_equal(vc[s], ovc)


def test_plain_q_without_gate_bf16_in_bf16_out(gpu_ctx, oracle):
    """cfg-3 style: bf16 activations, no gate, no norm, full rotary; Q and cache in bf16."""
    T, nh, nkv, hd = 5, 4, 2, 128
    q_in = rounded(oracle, oracle.randn((T, nh, hd), 17, 1), BF16)
    k_in = rounded(oracle, oracle.randn((T, nkv, hd), 17, 2), BF16)
    v_in = rounded(oracle, oracle.randn((T, nkv, hd), 17, 3), BF16)
    d_kc = torch.zeros((T, nkv, hd), dtype=torch.bfloat16, device="cuda")
    d_vc = torch.zeros_like(d_kc)
    d_q = torch.empty((T, nh, hd), dtype=torch.bfloat16, device="cuda")
    ops.kv_append_rope(gpu_ctx, q_proj_full=to_dev(q_in, BF16), k_proj=to_dev(k_in, BF16), v_proj=to_dev(v_in, BF16),
                       q_out=d_q, q_gate=None, cache=ops.KvCacheView(BF16, d_kc, d_vc, 0),
                       pos_start=torch.zeros(1, dtype=torch.int32).cuda(), num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                       rope_theta=1e6, rotary_dim=hd, num_seqs=1, tokens_per_seq=T, in_dtype=BF16, q_dtype=BF16,
                       has_gate=False, write_k_back=False)
    gpu_ctx.synchronize()
    okc, ovc = np.zeros((T, nkv, hd), np.float32), np.zeros((T, nkv, hd), np.float32)
    for j in range(T):
        qf = np.stack([q_in[j], np.zeros_like(q_in[j])], axis=1)
        oq, _, _ = oracle.fused_split_qknorm_kvstore(qf, k_in[j], v_in[j], okc, ovc, j, rope_theta=1e6, rotary_dim=hd)
        assert np.abs(to_host(d_q)[j] - oq).max() <= 2.0 ** -7 * np.abs(oq).max()
    assert np.abs(to_host(d_kc) - okc).max() <= 2.0 ** -7 * np.abs(okc).max()
    np.testing.assert_array_equal(to_host(d_vc), ovc)


@pytest.mark.parametrize("dt", [F16, BF16])
@pytest.mark.parametrize("hd,nh,nkv", [(128, 8, 2), (256, 4, 1)])
@pytest.mark.parametrize("write_k_back", [False, True])
def test_many_token_pass_equals_per_sequence_passes(gpu_ctx, oracle, dt, hd, nh, nkv, write_k_back):
    """A pass over enough tokens to give every warp one (rows staged through shared memory by bulk copies) against
    the same tokens appended one sequence per call (few enough tokens for the register kernel): bit for bit; and a
    few tokens against the oracle."""
    S, T, rd = 3, 512, hd // 4
    starts = [0, 37, 1000]
    rows = 1600
    q_in = rounded(oracle, oracle.randn((S, T, nh, hd), 23, 1), dt)
    k_in = rounded(oracle, oracle.randn((S, T, nkv, hd), 23, 2), dt)
    v_in = rounded(oracle, oracle.randn((S, T, nkv, hd), 23, 3), dt)
    w = oracle.bf16_bits(oracle.randn((2 * hd,), 23, 4) * np.float32(0.02))
    d_w = torch.from_numpy(w.view(np.int16)).cuda()

    def run(seqs, batched):
        d_kc = torch.zeros((S, rows, nkv, hd), dtype=TORCH_DT[dt], device="cuda")
        d_vc = torch.zeros_like(d_kc)
        d_q = torch.zeros((S, T, nh, hd), dtype=TORCH_DT[dt], device="cuda")
        d_k = to_dev(k_in, dt)
        d_qi, d_v = to_dev(q_in, dt), to_dev(v_in, dt)
        calls = [list(seqs)] if batched else [[s] for s in seqs]
        for group in calls:
            s0, n = group[0], len(group)
            ops.kv_append_rope(gpu_ctx, q_proj_full=d_qi[s0:s0 + n], k_proj=d_k[s0:s0 + n], v_proj=d_v[s0:s0 + n],
                               q_out=d_q[s0:s0 + n], q_gate=None,
                               cache=ops.KvCacheView(dt, d_kc[s0:s0 + n], d_vc[s0:s0 + n], rows * nkv * hd),
                               pos_start=torch.tensor(starts[s0:s0 + n], dtype=torch.int32).cuda(), num_heads=nh,
                               num_kv_heads=nkv, head_dim=hd, rope_theta=1e7, rotary_dim=rd, qk_norm_bf16=d_w,
                               num_seqs=n, tokens_per_seq=T, in_dtype=dt, q_dtype=dt, has_gate=False,
                               write_k_back=write_k_back)
        gpu_ctx.synchronize()
        return [t.view(torch.int16).cpu().numpy() for t in (d_q, d_k, d_kc, d_vc)], (d_q, d_kc)

    many, (d_q, d_kc) = run(range(S), True)
    each, _ = run(range(S), False)
    for a, b in zip(many, each):
        np.testing.assert_array_equal(a, b)
    if write_k_back:   # the rotated K went back over the projection
        np.testing.assert_array_equal(many[1].reshape(S, T, nkv, hd)[1], many[2][1, starts[1]:starts[1] + T])
    q, kc = to_host(d_q), to_host(d_kc)
    okc, ovc = np.zeros((rows, nkv, hd), np.float32), np.zeros((rows, nkv, hd), np.float32)
    for s, j in [(0, 0), (1, 300), (2, T - 1)]:
        qf = np.stack([q_in[s, j], np.zeros_like(q_in[s, j])], axis=1)
        oq, _, _ = oracle.fused_split_qknorm_kvstore(qf, k_in[s, j], v_in[s, j], okc, ovc, starts[s] + j, rope_theta=1e7,
                                                     rotary_dim=rd, qk_norm_bf16=w)
        assert np.abs(q[s, j] - oq).max() <= 2.0 ** -7 * np.abs(oq).max()
        assert np.abs(kc[s, starts[s] + j] - okc[starts[s] + j]).max() <= 2.0 ** -7 * np.abs(okc[starts[s] + j]).max()
