"""CPU tests of the oracle: closed forms, self-consistency, an independent formula, and the
committed fixtures.  The reference pins nothing numeric on this path, so this is all the
pinning the oracle can get."""
import importlib.util
import os

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _golden_module():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def _sdpa(q, k, v, L):
    nh, nkv = q.shape[0], k.shape[1]
    qt = torch.from_numpy(q).double()[None, :, None, :]
    kt = torch.from_numpy(k[:L]).double().permute(1, 0, 2).repeat_interleave(nh // nkv, 0)[None]
    vt = torch.from_numpy(v[:L]).double().permute(1, 0, 2).repeat_interleave(nh // nkv, 0)[None]
    return torch.nn.functional.scaled_dot_product_attention(qt, kt, vt)[0, :, 0, :].numpy()


def test_single_position_returns_v(oracle):
    q = oracle.randn((4, 64), 1, 1)
    k = oracle.randn((1, 2, 64), 1, 2)
    v = oracle.randn((1, 2, 64), 1, 3)
    out = oracle.gqa_attention_head(q, k, v, 1)
    np.testing.assert_array_equal(out, np.repeat(v[0], 2, axis=0))


def test_equal_keys_give_mean_of_v(oracle):
    q = oracle.randn((8, 128), 1, 1)
    k = np.broadcast_to(oracle.randn((1, 2, 128), 1, 2), (50, 2, 128)).copy()
    v = oracle.randn((50, 2, 128), 1, 3)
    out = oracle.gqa_attention_head(q, k, v, 50)
    np.testing.assert_allclose(out, np.repeat(v.mean(0), 4, axis=0), atol=2e-6)


@pytest.mark.parametrize("nh,nkv,hd,L", [(16, 2, 128, 512), (8, 8, 64, 33), (16, 2, 256, 300), (6, 2, 96, 17)])
def test_faithful_vs_f64_vs_sdpa(oracle, nh, nkv, hd, L):
    q, k, v = oracle.randn((nh, hd), 7, 1), oracle.randn((L + 3, nkv, hd), 7, 2), oracle.randn((L + 3, nkv, hd), 7, 3)
    o32 = oracle.gqa_attention_head(q, k, v, L)
    o64 = oracle.attention_f64(q, k, v, L)
    assert np.abs(o32 - o64).max() < 2e-6
    assert np.abs(o64 - _sdpa(q, k, v, L)).max() < 1e-12


@pytest.mark.parametrize("ns", [2, 3, 4, 7])
def test_split_plus_reduce_equals_single_pass(oracle, ns):
    nh, nkv, hd, L = 16, 2, 128, 203
    q, k, v = oracle.randn((nh, hd), 9, 1), oracle.randn((L, nkv, hd), 9, 2), oracle.randn((L, nkv, hd), 9, 3)
    one = oracle.gqa_attention_head(q, k, v, L)
    parts = oracle.gqa_attention_head(q, k, v, L, num_splits=ns)
    assert parts.shape == (nh, ns, hd + 2)
    np.testing.assert_allclose(oracle.gqa_reduce(parts), one, atol=2e-6)
    # [hd] = log(l) + m, [hd+1] = m  (gqa_attention_head.wgsl:120-121)
    assert np.all(parts[..., hd] >= parts[..., hd + 1])


def test_empty_split_poisons_verbatim_reduce_but_not_the_guarded_one(oracle):
    # ceil(5/4)=2 positions per split -> split 3 starts at 6 >= 5: empty (0/0, log 0)
    nh, nkv, hd, L = 4, 2, 64, 5
    q, k, v = oracle.randn((nh, hd), 3, 1), oracle.randn((L, nkv, hd), 3, 2), oracle.randn((L, nkv, hd), 3, 3)
    with np.errstate(all="ignore"):
        parts = oracle.gqa_attention_head(q, k, v, L, num_splits=4)
        assert np.isnan(parts[:, 3, :hd]).all()
        assert np.isnan(oracle.gqa_reduce(parts)).any()
        np.testing.assert_allclose(oracle.gqa_reduce(parts, skip_empty=True), oracle.gqa_attention_head(q, k, v, L),
                                   atol=2e-6)


def test_rope_position_zero_is_identity_and_gate_passes_through(oracle):
    nh, nkv, hd = 4, 2, 128
    qf, kp, vp = oracle.randn((nh, 2, hd), 5, 1), oracle.randn((nkv, hd), 5, 2), oracle.randn((nkv, hd), 5, 3)
    kc, vc = np.zeros((2, nkv, hd), np.float32), np.zeros((2, nkv, hd), np.float32)
    q, g, k = oracle.fused_split_qknorm_kvstore(qf, kp, vp, kc, vc, 0, rope_theta=1e6, rotary_dim=hd)
    np.testing.assert_array_equal(q, qf[:, 0])
    np.testing.assert_array_equal(g, qf[:, 1])
    np.testing.assert_array_equal(k, kp)
    np.testing.assert_array_equal(kc[0], kp)
    np.testing.assert_array_equal(vc[0], vp)
    assert not kc[1].any()


def test_rmsnorm_of_constant_vector(oracle):
    nh, nkv, hd = 2, 1, 128
    qf = np.full((nh, 2, hd), 3.0, np.float32)
    kp, vp = np.full((nkv, hd), -2.0, np.float32), np.zeros((nkv, hd), np.float32)
    kc, vc = np.zeros((1, nkv, hd), np.float32), np.zeros((1, nkv, hd), np.float32)
    w = np.zeros(2 * hd, np.uint16)  # weight 0 -> scale (1+0)
    q, _, k = oracle.fused_split_qknorm_kvstore(qf, kp, vp, kc, vc, 0, rope_theta=1e6, rotary_dim=0, qk_norm_bf16=w)
    np.testing.assert_allclose(q, 1.0, atol=1e-6)
    np.testing.assert_allclose(k, -1.0, atol=1e-6)


@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_matches_closed_form_and_preserves_norm(oracle, interleaved):
    nh, nkv, hd, rd, pos, theta = 2, 1, 128, 32, 77, 1e6
    qf, kp, vp = oracle.randn((nh, 2, hd), 6, 1), oracle.randn((nkv, hd), 6, 2), oracle.randn((nkv, hd), 6, 3)
    kc, vc = np.zeros((pos + 1, nkv, hd), np.float32), np.zeros((pos + 1, nkv, hd), np.float32)
    q, _, k = oracle.fused_split_qknorm_kvstore(qf, kp, vp, kc, vc, pos, rope_theta=theta, rotary_dim=rd,
                                                interleaved=interleaved)
    i = np.arange(rd // 2)
    ang = pos * theta ** (-2.0 * i / rd)
    x = qf[:, 0].astype(np.float64)
    want = x.copy()
    ia, ib = (2 * i, 2 * i + 1) if interleaved else (i, i + rd // 2)
    want[:, ia] = x[:, ia] * np.cos(ang) - x[:, ib] * np.sin(ang)
    want[:, ib] = x[:, ib] * np.cos(ang) + x[:, ia] * np.sin(ang)
    np.testing.assert_allclose(q, want, atol=5e-5)
    np.testing.assert_array_equal(q[:, rd:], qf[:, 0, rd:])  # dims >= rd pass through
    np.testing.assert_allclose(np.linalg.norm(k), np.linalg.norm(kp), rtol=1e-6)


def test_token_loop_equals_causal_attention(oracle):
    T, nh, nkv, hd = 40, 8, 2, 64
    q, k, v = oracle.randn((T, nh, hd), 11, 1), oracle.randn((T, nkv, hd), 11, 2), oracle.randn((T, nkv, hd), 11, 3)
    loop32 = oracle.causal_prefill(q, k, v)
    loop64 = oracle.causal_prefill(q, k, v, f64=True)
    qt = torch.from_numpy(q).double().permute(1, 0, 2)[None]
    kt = torch.from_numpy(k).double().permute(1, 0, 2).repeat_interleave(nh // nkv, 0)[None]
    vt = torch.from_numpy(v).double().permute(1, 0, 2).repeat_interleave(nh // nkv, 0)[None]
    ref = torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True)[0].permute(1, 0, 2).numpy()
    assert np.abs(loop64 - ref).max() < 1e-12
    assert np.abs(loop32 - ref).max() < 2e-6


def test_batched_decode_is_per_sequence_decode(oracle):
    nh, nkv, hd = 8, 2, 128
    lens = [5, 130, 1]
    q = oracle.randn((3, nh, hd), 13, 1)
    ks = [oracle.randn((L, nkv, hd), 13, 10 + i) for i, L in enumerate(lens)]
    vs = [oracle.randn((L, nkv, hd), 13, 20 + i) for i, L in enumerate(lens)]
    out = oracle.batched_decode(q, ks, vs, lens)
    for i, L in enumerate(lens):
        np.testing.assert_array_equal(out[i], oracle.gqa_attention_head(q[i], ks[i], vs[i], L))


def test_sigmoid_mul(oracle):
    x, g = oracle.randn((300,), 1, 1), oracle.randn((300,), 1, 2)
    np.testing.assert_allclose(oracle.sigmoid_mul(x, g), x / (1 + np.exp(-g.astype(np.float64))), rtol=1e-6)


def test_randn_is_counter_based_and_standard_normal(oracle):
    a = oracle.randn((100000,), 0x5EED, 7)
    b = oracle.randn((1000,), 0x5EED, 7, first_idx=500)
    np.testing.assert_array_equal(a[500:1500], b)
    assert abs(a.mean()) < 0.02 and abs(a.std() - 1) < 0.02
    assert not np.array_equal(a[:100], oracle.randn((100,), 0x5EED, 8))


def test_rounding_helpers_match_torch(oracle):
    x = oracle.randn((4096,), 2, 2) * np.float32(37.0)
    np.testing.assert_array_equal(oracle.round_bf16(x), torch.from_numpy(x).bfloat16().float().numpy())
    np.testing.assert_array_equal(oracle.round_f16(x), torch.from_numpy(x).half().float().numpy())


def test_golden_fixtures(oracle):
    g = _golden_module()
    gold = np.load(os.path.join(HERE, "golden", "golden_v1.npz"))
    np.testing.assert_array_equal(oracle.randn((16,), g.SEED, 1), gold["randn/first16"])
    for name in g.DECODE_CASES:
        r = g.run_decode(name)
        if isinstance(r, tuple):
            np.testing.assert_array_equal(r[0], gold[f"decode/{name}/partials"])
            np.testing.assert_array_equal(r[1], gold[f"decode/{name}/out"])
        else:
            np.testing.assert_array_equal(r, gold[f"decode/{name}/out"])
    for name in g.APPEND_CASES:
        for key, arr in zip(("q", "gate", "k", "k_row", "v_row"), g.run_append(name)):
            np.testing.assert_array_equal(arr, gold[f"append/{name}/{key}"])
