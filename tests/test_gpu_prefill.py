"""GPU parity of the causal prefill kernel (a-5: the batched form of the reference's token loop,
src/inference.rs:93-95) against the oracle's token loop in f64."""
import numpy as np
import pytest
import torch

from _util import RTOL_16, TORCH_DT, rel_err, rounded, to_dev, to_host
from shady_thinker_b200 import ops
from shady_thinker_b200._lib import BF16, F16, ShadyError

pytestmark = pytest.mark.gpu


def _run(gpu, oracle, B, T, nh, nkv, dt, seed, cap=None, hd=128):
    cap = cap or T
    q = rounded(oracle, oracle.randn((B, T, nh, hd), seed, 1), dt)
    k = rounded(oracle, oracle.randn((B, cap, nkv, hd), seed, 2), dt)
    v = rounded(oracle, oracle.randn((B, cap, nkv, hd), seed, 3), dt)
    d_out = torch.full((B, T, nh, hd), float("nan"), dtype=TORCH_DT[dt], device="cuda")
    view = ops.KvCacheView(dt, to_dev(k, dt), to_dev(v, dt), cap * nkv * hd)
    ops.attn_prefill(gpu, q=to_dev(q, dt), cache=view, out=d_out, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh,
                     num_seqs=B, seq_len=T, dtype=dt)
    gpu.synchronize()
    out = to_host(d_out)
    assert np.isfinite(out).all()
    for b in range(B):
        ref = oracle.causal_prefill(q[b], k[b, :T], v[b, :T], f64=True)
        # per-row check: early rows attend to few keys and have O(1) outputs, late rows are small
        err = np.abs(out[b] - ref).max(axis=(1, 2)) / np.abs(ref).max(axis=(1, 2))
        assert err.max() <= RTOL_16, (b, int(err.argmax()), float(err.max()))
    return out


@pytest.mark.parametrize("T", [128, 256, 384, 512])
def test_small_single_head(gpu_ctx, oracle, T):
    _run(gpu_ctx, oracle, 1, T, 1, 1, BF16, 11)


@pytest.mark.parametrize("dt", [BF16, F16])
def test_gqa_batch(gpu_ctx, oracle, dt):
    _run(gpu_ctx, oracle, 2, 640, 8, 2, dt, 12)


def test_ragged_length_and_padded_cache(gpu_ctx, oracle):
    # T not a multiple of the tile; cache capacity larger than T (rows >= T belong to the future)
    _run(gpu_ctx, oracle, 2, 333, 4, 2, BF16, 13, cap=400)
    _run(gpu_ctx, oracle, 1, 130, 4, 4, BF16, 14)


@pytest.mark.parametrize("T", [128, 192, 256, 333, 640])
def test_head_dim_256_small(gpu_ctx, oracle, T):
    """The wide-head kernel (one 128-row tile per item, 64-row K/V tiles, S double-buffered in TMEM)."""
    _run(gpu_ctx, oracle, 1, T, 2, 1, BF16, 21, hd=256)


@pytest.mark.parametrize("dt", [BF16, F16])
def test_head_dim_256_gqa_batch_more_items_than_sms(gpu_ctx, oracle, dt):
    # 3 x 16 heads x 5 row tiles = 240 items: every CTA walks more than one, the barrier phases run on through them
    _run(gpu_ctx, oracle, 3, 600, 16, 2, dt, 22, cap=640, hd=256)


def test_equals_decode_of_the_last_token(gpu_ctx, oracle):
    """Row T-1 of the prefill output == decode attention of that token over the same cache rows."""
    from _util import run_decode
    B, T, nh, nkv, hd, dt = 1, 1024, 8, 2, 128, BF16
    q = rounded(oracle, oracle.randn((B, T, nh, hd), 15, 1), dt)
    k = rounded(oracle, oracle.randn((B, T, nkv, hd), 15, 2), dt)
    v = rounded(oracle, oracle.randn((B, T, nkv, hd), 15, 3), dt)
    d_out = torch.empty((B, T, nh, hd), dtype=torch.bfloat16, device="cuda")
    view = ops.KvCacheView(dt, to_dev(k, dt), to_dev(v, dt), T * nkv * hd)
    ops.attn_prefill(gpu_ctx, q=to_dev(q, dt), cache=view, out=d_out, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh,
                     num_seqs=B, seq_len=T, dtype=dt)
    gpu_ctx.synchronize()
    dec = run_decode(gpu_ctx, q[:, T - 1], view, [T], nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=dt)
    assert rel_err(to_host(d_out)[0, T - 1], dec[0]) <= RTOL_16


def test_unsupported_shapes_return_status(gpu_ctx):
    d = torch.zeros(1024, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ShadyError) as e:
        ops.attn_prefill(gpu_ctx, q=d, cache=ops.KvCacheView(BF16, d, d, 0), out=d, head_dim=64, num_kv_heads=1,
                         num_q_heads=1, num_seqs=1, seq_len=8, dtype=BF16)
    assert e.value.code == 2


def test_cfg3_full_size_sampled_rows_and_linearity_in_v(gpu_ctx, oracle):
    """BASELINE config 3 at full size (B4, T4096, nh32/nkv8/hd128, bf16): sampled output rows against f64
    attention over the same rounded inputs, and two size-independent properties — doubling V doubles every output
    bit for bit (the softmax weights do not depend on V, and x2 is exact in bf16 and fp32), and a second run
    reproduces the first bit for bit."""
    B, T, nh, nkv, hd = 4, 4096, 32, 8, 128
    d_q = torch.empty((B, T, nh, hd), dtype=torch.bfloat16, device="cuda")
    d_k = torch.empty((B, T, nkv, hd), dtype=torch.bfloat16, device="cuda")
    d_v = torch.empty((B, T, nkv, hd), dtype=torch.bfloat16, device="cuda")
    ops.fill_randn(gpu_ctx, d_q, d_q.numel(), BF16, 0x5EED, 31)
    ops.fill_randn(gpu_ctx, d_k, d_k.numel(), BF16, 0x5EED, 32)
    ops.fill_randn(gpu_ctx, d_v, d_v.numel(), BF16, 0x5EED, 33)

    def run(v):
        d_out = torch.full((B, T, nh, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        view = ops.KvCacheView(BF16, d_k, v, T * nkv * hd)
        ops.attn_prefill(gpu_ctx, q=d_q, cache=view, out=d_out, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh,
                         num_seqs=B, seq_len=T, dtype=BF16)
        gpu_ctx.synchronize()
        return d_out

    out = run(d_v)
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out, run(d_v))
    assert torch.equal(run(d_v * 2), out * 2)
    # sampled (batch, row, head) triples: tile edges, the diagonal tiles, first and last rows
    rows = [0, 1, 127, 128, 129, 255, 256, 1000, 2047, 2048, 3071, 4000, 4094, 4095]
    scale = 1.0 / np.sqrt(hd)
    worst = 0.0
    for b in (0, 3):
        k = d_k[b].float().cpu().numpy().astype(np.float64)
        v = d_v[b].float().cpu().numpy().astype(np.float64)
        for r in rows:
            for h in (0, 5, 31):
                kvh = h // (nh // nkv)
                qv = d_q[b, r, h].float().cpu().numpy().astype(np.float64)
                s = (k[: r + 1, kvh] @ qv) * scale
                p = np.exp(s - s.max())
                ref = (p[:, None] * v[: r + 1, kvh]).sum(0) / p.sum()
                got = out[b, r, h].float().cpu().numpy()
                worst = max(worst, float(np.abs(got - ref).max() / np.abs(ref).max()))
    assert worst <= RTOL_16, worst


# ---- the prefill step from the projections: K/V append + Q norm/RoPE inside the attention kernel + gate ----------

def _fused_case(gpu, oracle, B, T, nh, nkv, dt, seed, rd, norm, gate, cap=None, hd=128):
    cap = cap or T
    qrow = 2 * hd if gate else hd
    qf = rounded(oracle, oracle.randn((B, T, nh, qrow), seed, 1), dt)
    kp = rounded(oracle, oracle.randn((B, T, nkv, hd), seed, 2), dt)
    vp = rounded(oracle, oracle.randn((B, T, nkv, hd), seed, 3), dt)
    w = oracle.bf16_bits(oracle.randn((2 * hd,), seed, 4) * np.float32(0.02)) if norm else None
    d_kc = torch.full((B, cap, nkv, hd), float("nan"), dtype=TORCH_DT[dt], device="cuda")
    d_vc = torch.full((B, cap, nkv, hd), float("nan"), dtype=TORCH_DT[dt], device="cuda")
    d_out = torch.full((B, T, nh, hd), float("nan"), dtype=TORCH_DT[dt], device="cuda")
    ws_n = ops.prefill_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_seqs=B, seq_len=T, dtype=dt)
    ws = torch.empty(ws_n, dtype=torch.uint8, device="cuda")
    ops.attn_prefill_append(gpu, q_proj_full=to_dev(qf, dt), k_proj=to_dev(kp, dt), v_proj=to_dev(vp, dt),
                            cache=ops.KvCacheView(dt, d_kc, d_vc, cap * nkv * hd), out=d_out, workspace=ws,
                            workspace_bytes=ws_n, num_heads=nh, num_kv_heads=nkv, head_dim=hd, num_seqs=B, seq_len=T,
                            rope_theta=1e6, rotary_dim=rd, dtype=dt,
                            qk_norm_bf16=torch.from_numpy(w.view(np.int16)).cuda() if norm else None, has_gate=gate)
    gpu.synchronize()
    out = to_host(d_out)
    assert np.isfinite(out).all()
    for b in range(B):
        # the oracle's token loop: append token t (norm, RoPE, cache rows), rows rounded to the cache dtype
        okc, ovc = np.zeros((T, nkv, hd), np.float32), np.zeros((T, nkv, hd), np.float32)
        oq = np.zeros((T, nh, hd), np.float32)
        og = np.zeros((T, nh, hd), np.float32)
        for t in range(T):
            full = qf[b, t].reshape(nh, 2, hd) if gate else np.stack([qf[b, t], np.zeros_like(qf[b, t])], 1)
            oq[t], og[t], _ = oracle.fused_split_qknorm_kvstore(full, kp[b, t], vp[b, t], okc, ovc, t, rope_theta=1e6,
                                                              rotary_dim=rd, qk_norm_bf16=w)
        okc, oq = rounded(oracle, okc, dt), rounded(oracle, oq, dt)
        got_k = to_host(d_kc[b, :T])
        assert np.abs(got_k - okc).max() <= 2.0 ** (-7 if dt == BF16 else -10) * np.abs(okc).max()
        np.testing.assert_array_equal(to_host(d_vc[b, :T]), vp[b])
        ref = oracle.causal_prefill(oq, okc, ovc, f64=True)
        if gate:
            ref = ref / (1.0 + np.exp(-og.astype(np.float64)))
        err = np.abs(out[b] - ref).max(axis=(1, 2)) / np.abs(ref).max(axis=(1, 2))
        assert err.max() <= RTOL_16, (b, int(err.argmax()), float(err.max()))
    if cap > T:      # rows past T were not touched
        assert torch.isnan(d_kc[:, T:].float()).all()


@pytest.mark.parametrize("rd,norm,gate", [(128, False, False), (32, True, True), (128, True, False), (64, False, True)])
def test_prefill_from_the_projections_matches_the_token_loop(gpu_ctx, oracle, rd, norm, gate):
    _fused_case(gpu_ctx, oracle, 2, 384, 8, 2, BF16, 51, rd, norm, gate)


@pytest.mark.parametrize("rd,norm,gate", [(64, True, True), (256, False, False)])
def test_prefill_from_the_projections_head_dim_256(gpu_ctx, oracle, rd, norm, gate):
    """The gated-attention layer shape: the step is one append pass (rotated Q into the workspace, K/V into the cache)
    and the wide-head attention kernel, whose epilogue applies the gate."""
    _fused_case(gpu_ctx, oracle, 2, 300, 4, 2, BF16, 55, rd, norm, gate, hd=256)


def test_prefill_from_the_projections_head_dim_256_many_tokens(gpu_ctx, oracle):
    """Enough tokens for the append pass to stage each token's rows through shared memory (Q heads fetched one by
    one past their gate halves)."""
    _fused_case(gpu_ctx, oracle, 2, 700, 4, 2, BF16, 56, 64, True, True, hd=256)


def test_prefill_from_the_projections_f16_ragged_and_many_items(gpu_ctx, oracle):
    _fused_case(gpu_ctx, oracle, 1, 333, 4, 2, F16, 52, 32, True, True, cap=400)
    # more items than SMs, so every CTA walks several and the three Q buffers rotate through their phases
    _fused_case(gpu_ctx, oracle, 3, 1100, 16, 4, BF16, 53, 32, True, True)


def test_prefill_from_the_projections_equals_the_two_calls(gpu_ctx, oracle):
    """Same step as shady_kv_append_rope followed by shady_attn_prefill (no gate): the cache rows are identical and
    the outputs agree to the rounding of the rotated Q."""
    B, T, nh, nkv, hd, dt = 2, 640, 8, 2, 128, BF16
    qf = to_dev(rounded(oracle, oracle.randn((B, T, nh, hd), 54, 1), dt), dt)
    kp = to_dev(rounded(oracle, oracle.randn((B, T, nkv, hd), 54, 2), dt), dt)
    vp = to_dev(rounded(oracle, oracle.randn((B, T, nkv, hd), 54, 3), dt), dt)
    outs, caches = [], []
    for fused in (False, True):
        d_kc = torch.zeros((B, T, nkv, hd), dtype=torch.bfloat16, device="cuda")
        d_vc = torch.zeros_like(d_kc)
        d_out = torch.zeros((B, T, nh, hd), dtype=torch.bfloat16, device="cuda")
        view = ops.KvCacheView(dt, d_kc, d_vc, T * nkv * hd)
        if fused:
            ws_n = ops.prefill_workspace_size(head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_seqs=B, seq_len=T)
            ws = torch.empty(ws_n, dtype=torch.uint8, device="cuda")
            ops.attn_prefill_append(gpu_ctx, q_proj_full=qf, k_proj=kp, v_proj=vp, cache=view, out=d_out, workspace=ws,
                                    workspace_bytes=ws_n, num_heads=nh, num_kv_heads=nkv, head_dim=hd, num_seqs=B,
                                    seq_len=T, rope_theta=1e6, rotary_dim=hd)
        else:
            d_q = torch.zeros((B, T, nh, hd), dtype=torch.bfloat16, device="cuda")
            ops.kv_append_rope(gpu_ctx, q_proj_full=qf, k_proj=kp.clone(), v_proj=vp, q_out=d_q, q_gate=None, cache=view,
                               pos_start=torch.zeros(B, dtype=torch.int32).cuda(), num_heads=nh, num_kv_heads=nkv,
                               head_dim=hd, rope_theta=1e6, rotary_dim=hd, num_seqs=B, tokens_per_seq=T, in_dtype=dt,
                               q_dtype=dt, has_gate=False, write_k_back=False)
            ops.attn_prefill(gpu_ctx, q=d_q, cache=view, out=d_out, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh,
                             num_seqs=B, seq_len=T, dtype=dt)
        gpu_ctx.synchronize()
        outs.append(to_host(d_out))
        caches.append((to_host(d_kc), to_host(d_vc)))
    np.testing.assert_array_equal(caches[0][0], caches[1][0])
    np.testing.assert_array_equal(caches[0][1], caches[1][1])
    # the two kernels may contract the rotation's multiply-adds differently: a Q element can land on the neighbouring
    # bf16 value, which moves an output by a fraction of its own rounding step
    assert rel_err(outs[1], outs[0]) <= 1e-2
    assert (outs[0] == outs[1]).mean() > 0.9
