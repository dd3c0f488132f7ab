"""GPU parity of the causal prefill kernel (a-5: the batched form of the reference's token loop,
src/inference.rs:93-95) against the oracle's token loop in f64."""
import numpy as np
import pytest
import torch

from _util import RTOL_16, TORCH_DT, rel_err, rounded, to_dev, to_host
from shady_thinker_b200 import ops
from shady_thinker_b200._lib import BF16, F16, ShadyError

pytestmark = pytest.mark.gpu


def _run(gpu, oracle, B, T, nh, nkv, dt, seed, cap=None):
    hd = 128
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
