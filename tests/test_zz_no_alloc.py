"""The workspace-free decode entry point (``shady_attn_decode_static``) against the regular one.

Some hosts of this library cannot allocate at call time — a server that has already given all device
memory to its KV-cache arena, or a decode loop that cannot take the device-wide stall of cudaMalloc —
so this variant keeps its scratch in a fixed 4 MiB array inside the library.  The file name sorts last
on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

from _util import RTOL_16, RaggedCache, rel_err, rounded, run_decode, to_dev, to_host
from shady_thinker_b200 import ops
from shady_thinker_b200._lib import BF16, F16, F32, ShadyError

pytestmark = pytest.mark.gpu


def _static_decode(gpu, q, view, lens, *, nh, nkv, hd, dt):
    S = len(lens)
    d_q = to_dev(q, dt)
    d_lens = torch.tensor(lens, dtype=torch.int32).cuda()
    d_out = torch.full((S, nh, hd), float("nan"), device="cuda")
    d_lse = torch.full((S, nh), float("nan"), device="cuda")
    ops.attn_decode_static(gpu, q=d_q, cache=view, seq_lens=d_lens, out=d_out, head_dim=hd, num_kv_heads=nkv,
                           num_q_heads=nh, num_seqs=S, num_splits=0, seq_lens_host=lens, q_dtype=dt, out_dtype=F32,
                           lse=d_lse)
    gpu.synchronize()
    return to_host(d_out), to_host(d_lse)


def test_two_calls_in_a_row_match_the_workspace_entry_point(gpu_ctx, oracle):
    nh, nkv, hd, dt = 32, 8, 128, F16
    for call, (seed, lens) in enumerate([(101, [700, 33, 1500, 16, 2049, 1]), (202, [3000, 5, 900, 1200, 64, 257])]):
        S = len(lens)
        q = rounded(oracle, oracle.randn((S, nh, hd), seed, 1), dt)
        ks = [rounded(oracle, oracle.randn((L, nkv, hd), seed, 10 + i), dt) for i, L in enumerate(lens)]
        vs = [rounded(oracle, oracle.randn((L, nkv, hd), seed, 50 + i), dt) for i, L in enumerate(lens)]
        cache = RaggedCache(ks, vs, dt)
        got, got_lse = _static_decode(gpu_ctx, q, cache.view, lens, nh=nh, nkv=nkv, hd=hd, dt=dt)
        want, want_lse = run_decode(gpu_ctx, q, cache.view, lens, nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=dt,
                                    out_dt=F32, want_lse=True)
        assert np.isfinite(got).all(), call
        for i in range(S):
            assert rel_err(got[i], want[i]) <= RTOL_16, (call, i)
        assert np.abs(got_lse - want_lse).max() <= 2e-2, call
        # and both agree with the oracle
        for i, L in enumerate(lens):
            assert rel_err(got[i], oracle.attention_f64(q[i], ks[i], vs[i], L)) <= RTOL_16, (call, i)


@pytest.mark.parametrize("dt,hd,nh,nkv,lens", [(BF16, 256, 16, 2, [40000]), (F16, 128, 8, 2, [30000, 100, 5000, 1])])
def test_long_sequences_are_merged_by_the_grid_as_in_the_workspace_entry_point(gpu_ctx, oracle, dt, hd, nh, nkv, lens):
    """A sequence cut into dozens of spans: both entry points plan the same launch (records merged by the whole
    grid after its barrier, one long sequence interleaved over all warps), here with the scratch in the built-in
    array; twice in a row, against the workspace form and the f64 oracle."""
    S = len(lens)
    q = rounded(oracle, oracle.randn((S, nh, hd), 303, 1), dt)
    ks = [rounded(oracle, oracle.randn((L, nkv, hd), 303, 10 + i), dt) for i, L in enumerate(lens)]
    vs = [rounded(oracle, oracle.randn((L, nkv, hd), 303, 50 + i), dt) for i, L in enumerate(lens)]
    cache = RaggedCache(ks, vs, dt)
    want, want_lse = run_decode(gpu_ctx, q, cache.view, lens, nh=nh, nkv=nkv, hd=hd, num_splits=0, q_dt=dt, out_dt=F32,
                                want_lse=True)
    for call in range(2):
        n0 = gpu_ctx.launch_count
        got, got_lse = _static_decode(gpu_ctx, q, cache.view, lens, nh=nh, nkv=nkv, hd=hd, dt=dt)
        assert gpu_ctx.launch_count - n0 == 1, "one cooperative launch, no second merge kernel"
        for i, L in enumerate(lens):
            assert rel_err(got[i], want[i]) <= 1e-5, (call, i)
            assert rel_err(got[i], oracle.attention_f64(q[i], ks[i], vs[i], L)) <= RTOL_16, (call, i)
        assert np.abs(got_lse - want_lse).max() <= 1e-5, call


def test_f32_cache_and_explicit_splits(gpu_ctx, oracle):
    nh, nkv, hd, L = 16, 2, 128, 512
    q, k, v = oracle.randn((1, nh, hd), 7, 1), oracle.randn((L, nkv, hd), 7, 2), oracle.randn((L, nkv, hd), 7, 3)
    view = ops.KvCacheView(F32, to_dev(k), to_dev(v), 0)
    d_lens = torch.tensor([L], dtype=torch.int32).cuda()
    for ns in (4, 0):
        d_out = torch.full((1, nh, hd), float("nan"), device="cuda")
        ops.attn_decode_static(gpu_ctx, q=to_dev(q), cache=view, seq_lens=d_lens, out=d_out, head_dim=hd,
                               num_kv_heads=nkv, num_q_heads=nh, num_seqs=1, num_splits=ns, seq_lens_host=[L])
        gpu_ctx.synchronize()
        assert np.abs(to_host(d_out)[0] - oracle.attention_f64(q[0], k, v, L)).max() <= 1e-3


def test_oversized_launch_is_refused_with_both_sizes_in_the_message(gpu_ctx):
    d = torch.zeros(64, device="cuda")
    lens = torch.ones(64, dtype=torch.int32, device="cuda")
    with pytest.raises(ShadyError) as e:   # 64 seqs x 64 splits x 32 heads x 130 floats = 68 MB of records
        ops.attn_decode_static(gpu_ctx, q=d, cache=ops.KvCacheView(F32, d, d, 0), seq_lens=lens, out=d, head_dim=128,
                               num_kv_heads=8, num_q_heads=32, num_seqs=64, num_splits=64)
    assert e.value.code == 4
    assert "4194304" in str(e.value) and "workspace" in str(e.value)
    gpu_ctx.synchronize()
