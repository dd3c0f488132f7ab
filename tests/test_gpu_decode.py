"""GPU parity of decode attention (a-1 + a-2) against the CPU oracle, through the C ABI."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from _util import ATOL_F32, RTOL_16, RaggedCache, rel_err, rounded, run_decode, to_dev, to_host
from shady_thinker_b200 import ops
from shady_thinker_b200._lib import BF16, F16, F32, ShadyError

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _golden_module():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def _single(oracle, nh, nkv, hd, L, seed, extra_rows=0):
    q = oracle.randn((nh, hd), seed, 1)
    k = oracle.randn((L + extra_rows, nkv, hd), seed, 2)
    v = oracle.randn((L + extra_rows, nkv, hd), seed, 3)
    return q, k, v


@pytest.mark.parametrize("ns", [1, 4, 0])
def test_cfg1_f32_against_oracle_and_golden(gpu_ctx, oracle, ns):
    g = _golden_module()
    nh, nkv, hd, L, _ = g.DECODE_CASES["cfg1_f32"]
    q, k, v = g.decode_inputs("cfg1_f32", nh, nkv, hd, L)
    view = ops.KvCacheView(F32, to_dev(k), to_dev(v), 0)
    out = run_decode(gpu_ctx, q[None], view, [L], nh=nh, nkv=nkv, hd=hd, num_splits=ns)[0]
    gold = np.load(os.path.join(HERE, "golden", "golden_v1.npz"))["decode/cfg1_f32/out"]
    assert np.abs(out - gold).max() <= ATOL_F32
    assert np.abs(out - oracle.attention_f64(q, k, v, L)).max() <= ATOL_F32


@pytest.mark.parametrize("nh,nkv,hd,L", [(16, 2, 128, 512), (4, 4, 64, 37), (16, 2, 256, 333), (6, 2, 128, 100)])
@pytest.mark.parametrize("ns", [2, 5])
def test_partials_layout_matches_reference_f32(gpu_ctx, oracle, nh, nkv, hd, L, ns):
    q, k, v = _single(oracle, nh, nkv, hd, L, 21)
    want = oracle.gqa_attention_head(q, k, v, L, num_splits=ns)
    d_part = torch.full((nh, ns, hd + 2), float("nan"), device="cuda")
    view = ops.KvCacheView(F32, to_dev(k), to_dev(v), 0)
    d_lens = torch.tensor([L], dtype=torch.int32).cuda()
    ops.attn_decode_partials(gpu_ctx, q=to_dev(q), cache=view, seq_lens=d_lens, partials=d_part, head_dim=hd,
                             num_kv_heads=nkv, num_q_heads=nh, num_splits=ns)
    gpu_ctx.synchronize()
    got = to_host(d_part)
    assert np.abs(got[..., :hd] - want[..., :hd]).max() <= ATOL_F32
    assert np.abs(got[..., hd] - want[..., hd]).max() <= ATOL_F32       # lse
    assert np.abs(got[..., hd + 1] - want[..., hd + 1]).max() <= ATOL_F32  # running max
    # a-2 through the C ABI on the oracle's own partials
    d_out = torch.empty((nh, hd), device="cuda")
    ops.attn_reduce(gpu_ctx, partials=to_dev(want), out=d_out, head_dim=hd, num_splits=ns, num_heads=nh)
    gpu_ctx.synchronize()
    assert np.abs(to_host(d_out) - oracle.gqa_reduce(want)).max() <= 1e-5


def test_reduce_skips_empty_splits(gpu_ctx, oracle):
    nh, nkv, hd, L, ns = 4, 2, 64, 5, 4   # split 3 is empty
    q, k, v = _single(oracle, nh, nkv, hd, L, 3)
    with np.errstate(all="ignore"):
        parts = oracle.gqa_attention_head(q, k, v, L, num_splits=ns)
    assert np.isnan(parts[:, 3, :hd]).all()
    d_out = torch.empty((nh, hd), device="cuda")
    ops.attn_reduce(gpu_ctx, partials=to_dev(parts), out=d_out, head_dim=hd, num_splits=ns, num_heads=nh)
    gpu_ctx.synchronize()
    assert np.abs(to_host(d_out) - oracle.attention_f64(q, k, v, L)).max() <= 1e-5
    # and the kernel's own empty splits carry lse = -inf, not NaN
    out = run_decode(gpu_ctx, q[None], ops.KvCacheView(F32, to_dev(k), to_dev(v), 0), [L], nh=nh, nkv=nkv, hd=hd,
                     num_splits=ns)[0]
    assert np.abs(out - oracle.attention_f64(q, k, v, L)).max() <= ATOL_F32


@pytest.mark.parametrize("dt", [F16, BF16])
@pytest.mark.parametrize("nh,nkv,hd", [(32, 8, 128), (16, 2, 256), (6, 2, 128), (32, 1, 128)])
@pytest.mark.parametrize("ns", [1, 3, 0])
def test_ragged_batch_16bit(gpu_ctx, oracle, dt, nh, nkv, hd, ns):
    lens = [1, 15, 16, 17, 0, 250, 1031]
    S = len(lens)
    q = rounded(oracle, oracle.randn((S, nh, hd), 31, 1), dt)
    ks = [rounded(oracle, oracle.randn((max(L, 1), nkv, hd), 31, 10 + i), dt) for i, L in enumerate(lens)]
    vs = [rounded(oracle, oracle.randn((max(L, 1), nkv, hd), 31, 50 + i), dt) for i, L in enumerate(lens)]
    cache = RaggedCache(ks, vs, dt)
    out, lse = run_decode(gpu_ctx, q, cache.view, lens, nh=nh, nkv=nkv, hd=hd, num_splits=ns, q_dt=dt, out_dt=F32,
                          want_lse=True)
    for i, L in enumerate(lens):
        if L == 0:
            assert not out[i].any() and np.isneginf(lse[i]).all()
            continue
        ref = oracle.attention_f64(q[i], ks[i], vs[i], L)
        assert rel_err(out[i], ref) <= RTOL_16, (i, L)
        # lse against f64
        G = nh // nkv
        s = np.einsum("hd,lhd->hl", q[i].astype(np.float64),
                      np.repeat(ks[i][:L].astype(np.float64), G, axis=1)) / np.sqrt(hd)
        ref_lse = np.log(np.exp(s - s.max(1, keepdims=True)).sum(1)) + s.max(1)
        assert np.abs(lse[i] - ref_lse).max() <= 2e-2


@pytest.mark.parametrize("dt,out_dt", [(F16, F16), (BF16, BF16)])
def test_16bit_output_dtype_and_strided_cache(gpu_ctx, oracle, dt, out_dt):
    nh, nkv, hd, S, Lmax = 16, 4, 128, 3, 700
    lens = [700, 123, 512]
    q = rounded(oracle, oracle.randn((S, nh, hd), 41, 1), dt)
    k = rounded(oracle, oracle.randn((S, Lmax, nkv, hd), 41, 2), dt)
    v = rounded(oracle, oracle.randn((S, Lmax, nkv, hd), 41, 3), dt)
    view = ops.KvCacheView(dt, to_dev(k, dt), to_dev(v, dt), Lmax * nkv * hd)
    out = run_decode(gpu_ctx, q, view, lens, nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=dt, out_dt=out_dt)
    for i, L in enumerate(lens):
        assert rel_err(out[i], oracle.attention_f64(q[i], k[i], v[i], L)) <= RTOL_16


def test_f32_query_with_16bit_cache(gpu_ctx, oracle):
    nh, nkv, hd, L = 16, 2, 128, 900
    q = oracle.randn((1, nh, hd), 43, 1)
    k = rounded(oracle, oracle.randn((L, nkv, hd), 43, 2), F16)
    v = rounded(oracle, oracle.randn((L, nkv, hd), 43, 3), F16)
    view = ops.KvCacheView(F16, to_dev(k, F16), to_dev(v, F16), 0)
    out = run_decode(gpu_ctx, q, view, [L], nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=F32, out_dt=F32)
    assert rel_err(out[0], oracle.attention_f64(q[0], k, v, L)) <= RTOL_16


@pytest.mark.parametrize("dt", [F32, F16])
def test_fused_gate_equals_sigmoid_mul_after(gpu_ctx, oracle, dt):
    nh, nkv, hd, L = 16, 2, 128, 300
    q = rounded(oracle, oracle.randn((1, nh, hd), 47, 1), dt)
    k = rounded(oracle, oracle.randn((L, nkv, hd), 47, 2), dt)
    v = rounded(oracle, oracle.randn((L, nkv, hd), 47, 3), dt)
    gate = oracle.randn((1, nh, hd), 47, 4)
    view = ops.KvCacheView(dt, to_dev(k, dt), to_dev(v, dt), 0)
    for ns in (1, 3):
        fused = run_decode(gpu_ctx, q, view, [L], nh=nh, nkv=nkv, hd=hd, num_splits=ns, q_dt=dt, gate=to_dev(gate))
        plain = run_decode(gpu_ctx, q, view, [L], nh=nh, nkv=nkv, hd=hd, num_splits=ns, q_dt=dt)
        want = oracle.sigmoid_mul(plain, gate).reshape(plain.shape)
        assert np.abs(fused - want).max() <= 1e-5
    # the stand-alone op (sigmoid_mul.wgsl)
    d_x = to_dev(plain)
    ops.sigmoid_mul(gpu_ctx, d_x, to_dev(gate), nh * hd)
    gpu_ctx.synchronize()
    assert np.abs(to_host(d_x) - want).max() <= 1e-6


def test_cfg2_shape_ragged_fp16_full_size(gpu_ctx, oracle):
    """BASELINE config 2: 32 sequences, L ~ U[1024, 8192], nh32/nkv8/hd128, fp16 KV + fp16 Q."""
    nh, nkv, hd, S = 32, 8, 128, 32
    rng = np.random.default_rng(0x5EED)
    lens = [int(x) for x in rng.integers(1024, 8193, S)]
    q = rounded(oracle, oracle.randn((S, nh, hd), 0x5EED, 1), F16)
    ks, vs = [], []
    for i, L in enumerate(lens):
        ks.append(rounded(oracle, oracle.randn((L, nkv, hd), 0x5EED, 100 + i), F16))
        vs.append(rounded(oracle, oracle.randn((L, nkv, hd), 0x5EED, 200 + i), F16))
    cache = RaggedCache(ks, vs, F16)
    out = run_decode(gpu_ctx, q, cache.view, lens, nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=F16, out_dt=F16)
    ref = oracle.batched_decode(q, ks, vs, lens)
    for i in range(S):
        assert rel_err(out[i], ref[i]) <= RTOL_16, (i, lens[i])


def test_long_context_bf16_hd256(gpu_ctx, oracle):
    """BASELINE config 4 shape at a length the oracle finishes quickly (nh16/nkv2/hd256, bf16)."""
    nh, nkv, hd, L = 16, 2, 256, 20000
    q = rounded(oracle, oracle.randn((1, nh, hd), 61, 1), BF16)
    k = rounded(oracle, oracle.randn((L, nkv, hd), 61, 2), BF16)
    v = rounded(oracle, oracle.randn((L, nkv, hd), 61, 3), BF16)
    view = ops.KvCacheView(BF16, to_dev(k, BF16), to_dev(v, BF16), 0)
    out = run_decode(gpu_ctx, q, view, [L], nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=BF16, out_dt=F32)
    assert rel_err(out[0], oracle.attention_f64(q[0], k, v, L, threads=8)) <= RTOL_16


def test_cfg4_full_size_against_f64_and_shard_merge(gpu_ctx, oracle):
    """BASELINE config 4 at full size (one sequence of 131072 rows, nh16/nkv2/hd256, bf16): three heads against
    f64 attention over the same device-filled rows, and a size-independent property — the rows cut into 8 shards,
    each decoded to (output, lse) records and merged rank-major, give the single-pass result."""
    nh, nkv, hd, L, P = 16, 2, 256, 131072, 8
    d_k = torch.empty((L, nkv, hd), dtype=torch.bfloat16, device="cuda")
    d_v = torch.empty((L, nkv, hd), dtype=torch.bfloat16, device="cuda")
    ops.fill_randn(gpu_ctx, d_k, d_k.numel(), BF16, 0x5EED, 41)
    ops.fill_randn(gpu_ctx, d_v, d_v.numel(), BF16, 0x5EED, 42)
    q = rounded(oracle, oracle.randn((1, nh, hd), 0x5EED, 43), BF16)
    view = ops.KvCacheView(BF16, d_k, d_v, 0)
    out = run_decode(gpu_ctx, q, view, [L], nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=BF16, out_dt=F32)[0]
    k = d_k.float().cpu().numpy()
    v = d_v.float().cpu().numpy()
    for h in (0, 7, 15):
        kvh = h // (nh // nkv)
        sc = (k[:, kvh].astype(np.float64) @ q[0, h].astype(np.float64)) / np.sqrt(hd)
        pr = np.exp(sc - sc.max())
        ref = (pr[:, None] * v[:, kvh]).sum(0) / pr.sum()
        assert rel_err(out[h], ref) <= RTOL_16, h
    recs = torch.zeros((P, nh, hd + 2), device="cuda")
    for r in range(P):
        lo, hi = r * L // P, (r + 1) * L // P
        sv = ops.KvCacheView(BF16, d_k[lo:hi], d_v[lo:hi], 0)
        o, lse = run_decode(gpu_ctx, q, sv, [hi - lo], nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=BF16, want_lse=True)
        recs[r, :, :hd] = torch.from_numpy(o[0]).cuda()
        recs[r, :, hd] = torch.from_numpy(lse[0]).cuda()
    d_out = torch.empty((nh, hd), device="cuda")
    ops.attn_reduce(gpu_ctx, partials=recs, out=d_out, head_dim=hd, num_splits=P, num_heads=nh,
                    split_stride=nh * (hd + 2), head_stride=hd + 2)
    gpu_ctx.synchronize()
    # both sides round P to bf16 over different row ranges: they agree to that rounding, not bit for bit
    err = rel_err(to_host(d_out), out)
    assert err <= 5e-3, err


def test_shards_merge_like_one_pass(gpu_ctx, oracle):
    """Split one sequence's rows over 4 'ranks', decode each shard with lse, merge rank-major records with
    shady_attn_reduce: equals the unsharded result (the cross-GPU combine run on one GPU)."""
    nh, nkv, hd, L, P = 16, 2, 256, 4096, 4
    q = rounded(oracle, oracle.randn((1, nh, hd), 71, 1), BF16)
    k = rounded(oracle, oracle.randn((L, nkv, hd), 71, 2), BF16)
    v = rounded(oracle, oracle.randn((L, nkv, hd), 71, 3), BF16)
    recs = torch.zeros((P, nh, hd + 2), device="cuda")
    bounds = [0, 1000, 1000, 3000, L]   # rank 1 is empty
    for r in range(P):
        lo, hi = bounds[r], bounds[r + 1]
        kk, vv = k[lo:max(hi, lo + 1)], v[lo:max(hi, lo + 1)]
        view = ops.KvCacheView(BF16, to_dev(kk, BF16), to_dev(vv, BF16), 0)
        o, lse = run_decode(gpu_ctx, q, view, [hi - lo], nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=BF16, want_lse=True)
        recs[r, :, :hd] = torch.from_numpy(o[0]).cuda()
        recs[r, :, hd] = torch.from_numpy(lse[0]).cuda()
    d_out = torch.empty((nh, hd), device="cuda")
    ops.attn_reduce(gpu_ctx, partials=recs, out=d_out, head_dim=hd, num_splits=P, num_heads=nh,
                    split_stride=nh * (hd + 2), head_stride=hd + 2)
    gpu_ctx.synchronize()
    assert rel_err(to_host(d_out), oracle.attention_f64(q[0], k, v, L)) <= RTOL_16


def test_bad_arguments_return_status_not_abort(gpu_ctx):
    d = torch.zeros(16, device="cuda")
    lens = torch.ones(1, dtype=torch.int32, device="cuda")
    view = ops.KvCacheView(F32, d, d, 0)
    with pytest.raises(ShadyError) as e:   # head_dim > 256: the shader's own limit
        ops.attn_decode(gpu_ctx, q=d, cache=view, seq_lens=lens, out=d, head_dim=512, num_kv_heads=1, num_q_heads=1,
                        num_splits=1)
    assert e.value.code == 2
    with pytest.raises(ShadyError) as e:   # nh not a multiple of nkv
        ops.attn_decode(gpu_ctx, q=d, cache=view, seq_lens=lens, out=d, head_dim=128, num_kv_heads=3, num_q_heads=4,
                        num_splits=1)
    assert e.value.code == 1
    with pytest.raises(ShadyError) as e:   # splits without a workspace
        ops.attn_decode(gpu_ctx, q=d, cache=view, seq_lens=lens, out=d, head_dim=128, num_kv_heads=1, num_q_heads=1,
                        num_splits=4)
    assert e.value.code == 4
    gpu_ctx.synchronize()   # the context is still usable


def test_decode_shard_records_merge_rank_major(gpu_ctx, oracle):
    """shady_attn_decode_shard on each 'rank' range of one sequence + the rank-major merge == unsharded decode."""
    from shady_thinker_b200.sharding import merge_args, shard_rows
    nh, nkv, hd, L, P = 16, 2, 256, 5000, 4
    q = rounded(oracle, oracle.randn((1, nh, hd), 73, 1), BF16)
    k = rounded(oracle, oracle.randn((L, nkv, hd), 73, 2), BF16)
    v = rounded(oracle, oracle.randn((L, nkv, hd), 73, 3), BF16)
    gathered = torch.full((P, 1, nh, hd + 2), float("nan"), device="cuda")
    ws_n = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=0, num_seqs=1)
    ws = torch.zeros(ws_n, dtype=torch.uint8, device="cuda")
    d_q = to_dev(q, BF16)
    for r in range(P):
        lo, hi = shard_rows(L, P, r)
        kk, vv = k[lo:max(hi, lo + 1)], v[lo:max(hi, lo + 1)]
        view = ops.KvCacheView(BF16, to_dev(kk, BF16), to_dev(vv, BF16), 0)
        lens = torch.tensor([hi - lo], dtype=torch.int32).cuda()
        ops.attn_decode_shard(gpu_ctx, q=d_q, cache=view, seq_lens=lens, records=gathered[r], head_dim=hd,
                              num_kv_heads=nkv, num_q_heads=nh, num_seqs=1, num_splits=0, seq_lens_host=[hi - lo],
                              q_dtype=BF16, workspace=ws, workspace_bytes=ws_n)
        gpu_ctx.synchronize()
    d_out = torch.empty((nh, hd), device="cuda")
    ops.attn_reduce(gpu_ctx, partials=gathered, out=d_out, **merge_args(1, nh, hd, P))
    gpu_ctx.synchronize()
    assert rel_err(to_host(d_out), oracle.attention_f64(q[0], k, v, L)) <= RTOL_16
    # an empty shard: lse = -inf, zeros
    view = ops.KvCacheView(BF16, to_dev(k[:1], BF16), to_dev(v[:1], BF16), 0)
    rec = torch.full((1, nh, hd + 2), float("nan"), device="cuda")
    ops.attn_decode_shard(gpu_ctx, q=d_q, cache=view, seq_lens=torch.zeros(1, dtype=torch.int32).cuda(), records=rec,
                          head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_seqs=1, num_splits=0, seq_lens_host=[0],
                          q_dtype=BF16, workspace=ws, workspace_bytes=ws_n)
    gpu_ctx.synchronize()
    rh = to_host(rec)
    assert np.isneginf(rh[0, :, hd]).all() and not rh[0, :, :hd].any()


@pytest.mark.parametrize("lens", [[1, 16, 17, 700, 2500, 33], [20000, 50]], ids=["short", "deferred-merge"])
@pytest.mark.parametrize("dt,in_dt,norm,gate,rd", [(F16, F16, False, False, 128), (BF16, F32, True, True, 32),
                                                   (F16, F32, True, False, 64)])
def test_fused_append_decode_equals_the_two_calls(gpu_ctx, oracle, dt, in_dt, norm, gate, rd, lens):
    """shady_attn_decode_append == shady_kv_append_rope followed by shady_attn_decode (+ gate), cache rows included."""
    from _util import TORCH_DT
    nh, nkv, hd = 32, 8, 128
    S = len(lens)                                          # lengths INCLUDE the appended token
    qmul = 2 if gate else 1
    q_full = rounded(oracle, oracle.randn((S, nh, qmul * hd), 81, 1), in_dt)
    k_new = rounded(oracle, oracle.randn((S, nkv, hd), 81, 2), in_dt)
    v_new = rounded(oracle, oracle.randn((S, nkv, hd), 81, 3), in_dt)
    w = oracle.bf16_bits(oracle.randn((2 * hd,), 81, 4) * np.float32(0.02)) if norm else None
    d_w = torch.from_numpy(w.view(np.int16)).cuda() if norm else None
    ks = [rounded(oracle, oracle.randn((L, nkv, hd), 81, 10 + i), dt) for i, L in enumerate(lens)]
    vs = [rounded(oracle, oracle.randn((L, nkv, hd), 81, 50 + i), dt) for i, L in enumerate(lens)]
    d_lens = torch.tensor(lens, dtype=torch.int32).cuda()
    d_pos = torch.tensor([L - 1 for L in lens], dtype=torch.int32).cuda()
    ws_n = ops.decode_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_splits=0, num_seqs=S)
    ws = torch.zeros(ws_n, dtype=torch.uint8, device="cuda")
    # --- reference: two calls ---
    c1 = RaggedCache(ks, vs, dt)
    d_q = torch.empty((S, nh, hd), dtype=TORCH_DT[in_dt], device="cuda")
    d_g = torch.empty((S, nh, hd), device="cuda") if gate else None
    ops.kv_append_rope(gpu_ctx, q_proj_full=to_dev(q_full, in_dt), k_proj=to_dev(k_new, in_dt), v_proj=to_dev(v_new, in_dt),
                       q_out=d_q, q_gate=d_g, cache=c1.view, pos_start=d_pos, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                       rope_theta=1e6, rotary_dim=rd, qk_norm_bf16=d_w, num_seqs=S, in_dtype=in_dt, q_dtype=in_dt,
                       has_gate=gate, write_k_back=False)
    want = torch.empty((S, nh, hd), device="cuda")
    ops.attn_decode(gpu_ctx, q=d_q, cache=c1.view, seq_lens=d_lens, out=want, head_dim=hd, num_kv_heads=nkv,
                    num_q_heads=nh, num_seqs=S, num_splits=0, seq_lens_host=lens, q_dtype=in_dt, gate=d_g, workspace=ws,
                    workspace_bytes=ws_n)
    gpu_ctx.synchronize()
    # --- fused: one call on a fresh copy of the caches ---
    c2 = RaggedCache(ks, vs, dt)
    got = torch.full((S, nh, hd), float("nan"), device="cuda")
    ops.attn_decode_append(gpu_ctx, q_proj_full=to_dev(q_full, in_dt), k_proj=to_dev(k_new, in_dt),
                           v_proj=to_dev(v_new, in_dt), cache=c2.view, seq_lens=d_lens, out=got, num_heads=nh,
                           num_kv_heads=nkv, head_dim=hd, rope_theta=1e6, rotary_dim=rd, num_seqs=S, qk_norm_bf16=d_w,
                           in_dtype=in_dt, has_gate=gate, seq_lens_host=lens, workspace=ws, workspace_bytes=ws_n)
    gpu_ctx.synchronize()
    for i, L in enumerate(lens):
        ulp = 2.0 ** -10 if dt == F16 else 2.0 ** -7       # the two kernels may contract their FMAs differently
        k1, k2 = to_host(c1.k[i])[L - 1], to_host(c2.k[i])[L - 1]
        assert np.abs(k2 - k1).max() <= ulp * np.abs(k1).max(), (i, L)
        np.testing.assert_array_equal(to_host(c2.v[i])[L - 1], to_host(c1.v[i])[L - 1])   # V is a pure copy
        np.testing.assert_array_equal(to_host(c2.k[i])[:L - 1], ks[i][:L - 1])            # older rows untouched
        # Q is rounded to the cache dtype when staged in both paths only if in_dt == dt; allow the 16-bit tolerance
        assert rel_err(to_host(got)[i], to_host(want)[i]) <= RTOL_16, (i, L)


@pytest.mark.parametrize("dt,nh,nkv,hd,lens", [(BF16, 16, 2, 256, [40000]), (F16, 32, 8, 128, [30000, 100, 5000, 1])])
def test_merge_by_the_decode_grid_equals_the_second_launch(oracle, monkeypatch, dt, nh, nkv, hd, lens):
    """Sequences cut into more spans than their last CTA merges alone: by default the decode grid meets at a barrier
    and merges the records itself (one cooperative launch; the blocks of a single long sequence are also interleaved
    over all warps, SHADY_DECODE_INTERLEAVE=0 keeps fixed spans); SHADY_DECODE_GRID_MERGE=0 keeps the second launch.
    All must give the reference's merge (gqa_reduce.wgsl:33-64) of the same rows, gate included, launch after launch
    (the barrier words zero themselves).  The knobs are read when a context is created, hence one context each."""
    from shady_thinker_b200.gpu import GpuContext
    S = len(lens)
    q = rounded(oracle, oracle.randn((S, nh, hd), 71, 1), dt)
    gate = torch.from_numpy(oracle.randn((S, nh, hd), 71, 2)).cuda()
    ks = [rounded(oracle, oracle.randn((L, nkv, hd), 71, 10 + i), dt) for i, L in enumerate(lens)]
    vs = [rounded(oracle, oracle.randn((L, nkv, hd), 71, 50 + i), dt) for i, L in enumerate(lens)]
    cache = RaggedCache(ks, vs, dt)

    def runs(ctx, n):
        n0 = ctx.launch_count
        outs = [run_decode(ctx, q, cache.view, lens, nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=dt, out_dt=F32,
                           want_lse=True, gate=gate) for _ in range(n)]
        return outs, ctx.launch_count - n0

    def same_bits(outs):
        for o, l in outs[1:]:
            np.testing.assert_array_equal(o, outs[0][0])
            np.testing.assert_array_equal(l, outs[0][1])

    with GpuContext(0, stream=0x1) as ctx:                       # defaults: a single long sequence is interleaved
        ilv, launches = runs(ctx, 3)
        assert launches == 3                                     # one launch per decode
    same_bits(ilv)
    monkeypatch.setenv("SHADY_DECODE_INTERLEAVE", "0")
    with GpuContext(0, stream=0x1) as ctx:                       # fixed spans
        outs, launches = runs(ctx, 3)
        assert launches == 3
    same_bits(outs)
    monkeypatch.setenv("SHADY_DECODE_GRID_MERGE", "0")
    with GpuContext(0, stream=0x1) as ctx:
        (two_pair,), launches = runs(ctx, 1)
        assert launches == 2
    two, two_lse = two_pair
    one, one_lse = outs[0]
    assert np.abs(one - two).max() <= 2e-6 * max(1.0, np.abs(two).max())
    assert np.abs(one_lse - two_lse).max() <= 1e-5
    # interleaved, a warp sees other rows than in its span: its running maximum, and with it the 16-bit rounding of P, differs
    assert np.abs(ilv[0][0] - two).max() <= 5e-3 * np.abs(two).max()
    assert np.abs(ilv[0][1] - two_lse).max() <= 1e-3
    sig = 1.0 / (1.0 + np.exp(-to_host(gate).astype(np.float64)))
    for i, L in enumerate(lens):
        want = oracle.attention_f64(q[i], ks[i], vs[i], L, threads=8) * sig[i]
        assert rel_err(one[i], want) <= RTOL_16, (i, L)
