"""Causal prefill of a LISTED batch — prompts of different lengths packed token-major — over caches of every
addressing the library knows (one allocation with a stride, per-sequence pointer arrays, page pools behind a page
table), against the oracle's token loop in f64 (the reference prefills every cache slot, model.rs:973-1029, through
its own loop, inference.rs:93-95).  Memory past a sequence's end is poisoned with NaN wherever the entry point
promises not to let it reach a result."""
import numpy as np
import pytest
import torch

from _util import RTOL_16, TORCH_DT, rel_err, rounded, to_dev, to_host
from shady_thinker_b200 import ops
from shady_thinker_b200._lib import BF16, F16, ShadyError
from shady_thinker_b200.paged import PagedKvCache

pytestmark = pytest.mark.gpu
NAN = float("nan")


def _check_rows(out, ref, tag):
    err = np.abs(out - ref).max(axis=(1, 2)) / np.abs(ref).max(axis=(1, 2))
    assert err.max() <= RTOL_16, (tag, int(err.argmax()), float(err.max()))


def _paged(gpu, lens, page_rows, nkv, hd, dt, seed, poison):
    """A pool whose pages are handed out in shuffled order; rows no sequence owns hold ``poison``."""
    S = len(lens)
    need = sum((L + page_rows - 1) // page_rows for L in lens)
    pc = PagedKvCache(gpu, num_seqs=S, num_pages=need + 2, page_rows=page_rows, num_kv_heads=nkv, head_dim=hd,
                      kv_dtype=dt, max_pages_per_seq=max((L + page_rows - 1) // page_rows for L in lens))
    rng = np.random.default_rng(seed)
    rng.shuffle(pc.free)
    for s in rng.permutation(S):
        pc.ensure(int(s), lens[int(s)])
    n = pc.num_pages * page_rows * nkv * hd
    kp = torch.full((n,), poison, dtype=TORCH_DT[dt], device="cuda")
    vp = torch.full((n,), poison, dtype=TORCH_DT[dt], device="cuda")
    return pc, kp, vp


def _store_pool(pc, kp, vp):
    pc.gpu.copy_buffer(kp, pc.k_pool, kp.numel() * 2)
    pc.gpu.copy_buffer(vp, pc.v_pool, vp.numel() * 2)
    pc.gpu.synchronize()


def _scatter(pc, pool, s, rows, dt):
    row = pc.nkv * pc.hd
    d = to_dev(rows, dt).reshape(-1)
    for r0 in range(0, rows.shape[0], pc.page_rows):
        n = min(pc.page_rows, rows.shape[0] - r0)
        off = pc.row_offset(s, r0)
        pool[off:off + n * row] = d[r0 * row:(r0 + n) * row]


def _plain_case(gpu, oracle, lens, nh, nkv, hd, dt, seed, layout, page_rows=0):
    S, tot = len(lens), sum(lens)
    q = rounded(oracle, oracle.randn((tot, nh, hd), seed, 1), dt)
    ks = [rounded(oracle, oracle.randn((L, nkv, hd), seed, 10 + s), dt) for s, L in enumerate(lens)]
    vs = [rounded(oracle, oracle.randn((L, nkv, hd), seed, 100 + s), dt) for s, L in enumerate(lens)]
    keep, kw = [], {}
    if layout == "stride":      # one allocation, capacity rows per sequence, rows past T_i poisoned
        cap = max(lens) + 37
        d_k = torch.full((S, cap, nkv, hd), NAN, dtype=TORCH_DT[dt], device="cuda")
        d_v = torch.full((S, cap, nkv, hd), NAN, dtype=TORCH_DT[dt], device="cuda")
        for s, L in enumerate(lens):
            d_k[s, :L], d_v[s, :L] = to_dev(ks[s], dt), to_dev(vs[s], dt)
        view = ops.KvCacheView(dt, d_k, d_v, cap * nkv * hd)
    elif layout == "ptrs":      # every sequence its own allocation of exactly T_i rows
        keep = [[to_dev(k, dt) for k in ks], [to_dev(v, dt) for v in vs]]
        kp = [t.data_ptr() for t in keep[0]]
        vp = [t.data_ptr() for t in keep[1]]
        view = ops.KvCacheView(dt, k_ptrs=torch.tensor(kp, dtype=torch.int64).cuda(), v_ptrs=torch.tensor(vp, dtype=torch.int64).cuda())
        kw = dict(k_ptrs=kp, v_ptrs=vp)
    else:                       # pages; the pool is initialised (zero), as the entry point asks
        pc, kpool, vpool = _paged(gpu, lens, page_rows, nkv, hd, dt, seed, 0.0)
        for s in range(S):
            _scatter(pc, kpool, s, ks[s], dt)
            _scatter(pc, vpool, s, vs[s], dt)
        _store_pool(pc, kpool, vpool)
        view = pc.view
    ws_n = ops.prefill_ragged_workspace_size(seq_lens=lens, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, dtype=dt)
    ws = torch.empty(ws_n, dtype=torch.uint8, device="cuda")
    d_out = torch.full((tot, nh, hd), NAN, dtype=TORCH_DT[dt], device="cuda")
    ops.attn_prefill_ragged(gpu, q=to_dev(q, dt), cache=view, out=d_out, seq_lens=lens, workspace=ws, workspace_bytes=ws_n,
                            head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, dtype=dt, **kw)
    gpu.synchronize()
    out = to_host(d_out)
    assert np.isfinite(out).all()
    t0 = 0
    for s, L in enumerate(lens):
        _check_rows(out[t0:t0 + L], oracle.causal_prefill(q[t0:t0 + L], ks[s], vs[s], f64=True), (layout, s))
        t0 += L
    return out


LENS = [300, 1, 129, 515, 256, 64]


@pytest.mark.parametrize("layout", ["stride", "ptrs"])
@pytest.mark.parametrize("hd", [128, 256])
def test_listed_batch_one_map_per_sequence(gpu_ctx, oracle, layout, hd):
    _plain_case(gpu_ctx, oracle, LENS, 4, 2, hd, BF16, 61, layout)


@pytest.mark.parametrize("hd,page_rows", [(128, 16), (128, 64), (128, 128), (128, 256), (256, 16), (256, 64), (256, 192)])
def test_listed_batch_paged(gpu_ctx, oracle, hd, page_rows):
    _plain_case(gpu_ctx, oracle, LENS, 4, 2, hd, F16, 62, "paged", page_rows)


def test_more_row_blocks_than_sms(gpu_ctx, oracle):
    # 5 sequences x (2..5 row blocks) x 16 heads: every CTA walks several items of different sequences
    _plain_case(gpu_ctx, oracle, [1100, 700, 513, 1025, 900], 16, 4, 128, BF16, 63, "ptrs")


def test_equal_lengths_give_the_bytes_of_the_uniform_call(gpu_ctx, oracle):
    B, T, nh, nkv, hd, dt = 3, 640, 8, 2, 128, BF16
    q = to_dev(rounded(oracle, oracle.randn((B, T, nh, hd), 64, 1), dt), dt)
    k = to_dev(rounded(oracle, oracle.randn((B, T, nkv, hd), 64, 2), dt), dt)
    v = to_dev(rounded(oracle, oracle.randn((B, T, nkv, hd), 64, 3), dt), dt)
    view = ops.KvCacheView(dt, k, v, T * nkv * hd)
    a = torch.zeros((B, T, nh, hd), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((B * T, nh, hd), dtype=torch.bfloat16, device="cuda")
    ops.attn_prefill(gpu_ctx, q=q, cache=view, out=a, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, num_seqs=B, seq_len=T, dtype=dt)
    ws_n = ops.prefill_ragged_workspace_size(seq_lens=[T] * B, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, dtype=dt)
    ws = torch.empty(ws_n, dtype=torch.uint8, device="cuda")
    ops.attn_prefill_ragged(gpu_ctx, q=q, cache=view, out=b, seq_lens=[T] * B, workspace=ws, workspace_bytes=ws_n,
                            head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, dtype=dt)
    gpu_ctx.synchronize()
    assert torch.equal(a.reshape(B * T, nh, hd), b)


# ---- the step from the projections ----------------------------------------------------------------------------

def _fused_case(gpu, oracle, lens, nh, nkv, hd, dt, seed, rd, layout, page_rows=0, gate=True):
    S, tot = len(lens), sum(lens)
    qrow = 2 * hd if gate else hd
    qf = rounded(oracle, oracle.randn((tot, nh, qrow), seed, 1), dt)
    kp = rounded(oracle, oracle.randn((tot, nkv, hd), seed, 2), dt)
    vp = rounded(oracle, oracle.randn((tot, nkv, hd), seed, 3), dt)
    w = oracle.bf16_bits(oracle.randn((2 * hd,), seed, 4) * np.float32(0.02))
    keep, kw, pc = [], {}, None
    if layout == "stride":
        cap = max(lens) + 5
        d_k = torch.full((S, cap, nkv, hd), NAN, dtype=TORCH_DT[dt], device="cuda")
        d_v = torch.full((S, cap, nkv, hd), NAN, dtype=TORCH_DT[dt], device="cuda")
        view = ops.KvCacheView(dt, d_k, d_v, cap * nkv * hd)
        rows = lambda t, s, L: to_host(t[s, :L])
        keep = [d_k, d_v]
    elif layout == "ptrs":
        keep = [[torch.full((L, nkv, hd), NAN, dtype=TORCH_DT[dt], device="cuda") for L in lens] for _ in range(2)]
        kps, vps = [t.data_ptr() for t in keep[0]], [t.data_ptr() for t in keep[1]]
        view = ops.KvCacheView(dt, k_ptrs=torch.tensor(kps, dtype=torch.int64).cuda(), v_ptrs=torch.tensor(vps, dtype=torch.int64).cuda())
        kw = dict(k_ptrs=kps, v_ptrs=vps)
        rows = lambda t, s, L: to_host(t[s])
    else:   # pages that an earlier owner left full of NaN: the step clears what travels with the last tile
        pc, kpool, vpool = _paged(gpu, lens, page_rows, nkv, hd, dt, seed, NAN)
        _store_pool(pc, kpool, vpool)
        view = pc.view
    ws_n = ops.prefill_ragged_workspace_size(seq_lens=lens, head_dim=hd, num_kv_heads=nkv, num_q_heads=nh, dtype=dt, with_append=True)
    ws = torch.empty(ws_n, dtype=torch.uint8, device="cuda")
    d_out = torch.full((tot, nh, hd), NAN, dtype=TORCH_DT[dt], device="cuda")
    ops.attn_prefill_append_ragged(gpu, q_proj_full=to_dev(qf, dt), k_proj=to_dev(kp, dt), v_proj=to_dev(vp, dt), cache=view,
                                   out=d_out, seq_lens=lens, workspace=ws, workspace_bytes=ws_n, num_heads=nh, num_kv_heads=nkv,
                                   head_dim=hd, rope_theta=1e6, rotary_dim=rd, dtype=dt,
                                   qk_norm_bf16=torch.from_numpy(w.view(np.int16)).cuda(), has_gate=gate, **kw)
    gpu.synchronize()
    out = to_host(d_out)
    assert np.isfinite(out).all()
    if pc is not None:
        pool_k = torch.empty(pc.num_pages * page_rows * nkv * hd, dtype=TORCH_DT[dt], device="cuda")
        pool_v = torch.empty_like(pool_k)
        gpu.copy_buffer(pc.k_pool, pool_k, pool_k.numel() * 2)
        gpu.copy_buffer(pc.v_pool, pool_v, pool_v.numel() * 2)
        gpu.synchronize()

        def rows(which, s, L):
            pool, row = (pool_k, pool_v)[which], nkv * hd
            return to_host(torch.stack([pool[pc.row_offset(s, r):pc.row_offset(s, r) + row] for r in range(L)]).reshape(L, nkv, hd))
    t0 = 0
    for s, L in enumerate(lens):
        okc, ovc = np.zeros((L, nkv, hd), np.float32), np.zeros((L, nkv, hd), np.float32)
        oq, og = np.zeros((L, nh, hd), np.float32), np.zeros((L, nh, hd), np.float32)
        for t in range(L):
            full = qf[t0 + t].reshape(nh, 2, hd) if gate else np.stack([qf[t0 + t], np.zeros_like(qf[t0 + t])], 1)
            oq[t], og[t], _ = oracle.fused_split_qknorm_kvstore(full, kp[t0 + t], vp[t0 + t], okc, ovc, t, rope_theta=1e6,
                                                              rotary_dim=rd, qk_norm_bf16=w)
        okc, oq = rounded(oracle, okc, dt), rounded(oracle, oq, dt)
        got_k = rows(0, s, L) if pc is not None else rows(keep[0], s, L)
        got_v = rows(1, s, L) if pc is not None else rows(keep[1], s, L)
        assert np.abs(got_k - okc).max() <= 2.0 ** (-7 if dt == BF16 else -10) * np.abs(okc).max(), s
        np.testing.assert_array_equal(got_v, vp[t0:t0 + L])
        ref = oracle.causal_prefill(oq, okc, ovc, f64=True)
        if gate:
            ref = ref / (1.0 + np.exp(-og.astype(np.float64)))
        _check_rows(out[t0:t0 + L], ref, (layout, s))
        t0 += L
    if layout == "stride":      # rows past every sequence's end were not touched
        for s, L in enumerate(lens):
            assert torch.isnan(keep[0][s, L:].float()).all()


FLENS = [200, 37, 130, 1, 260]


@pytest.mark.parametrize("layout,page_rows", [("stride", 0), ("ptrs", 0), ("paged", 32), ("paged", 128)])
def test_step_from_the_projections_listed(gpu_ctx, oracle, layout, page_rows):
    _fused_case(gpu_ctx, oracle, FLENS, 4, 2, 128, BF16, 71, 32, layout, page_rows)


@pytest.mark.parametrize("layout,page_rows", [("ptrs", 0), ("paged", 64)])
def test_step_from_the_projections_listed_head_dim_256(gpu_ctx, oracle, layout, page_rows):
    _fused_case(gpu_ctx, oracle, FLENS, 4, 2, 256, F16, 72, 64, layout, page_rows)


def test_bad_batches_return_a_status(gpu_ctx):
    d = torch.zeros(1 << 16, dtype=torch.bfloat16, device="cuda")
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    base = dict(q=d, out=d, workspace=ws, workspace_bytes=ws.numel(), head_dim=128, num_kv_heads=1, num_q_heads=1, dtype=BF16)
    with pytest.raises(ShadyError) as e:      # an empty sequence
        ops.attn_prefill_ragged(gpu_ctx, cache=ops.KvCacheView(BF16, d, d, 4096), seq_lens=[16, 0], **base)
    assert e.value.code == 1
    with pytest.raises(ShadyError) as e:      # workspace smaller than the size call says
        ops.attn_prefill_ragged(gpu_ctx, cache=ops.KvCacheView(BF16, d, d, 4096), seq_lens=[16, 8],
                                **{**base, "workspace_bytes": 64})
    assert e.value.code == 4
    ptrs = torch.tensor([d.data_ptr()], dtype=torch.int64).cuda()
    with pytest.raises(ShadyError) as e:      # pointer-array cache without the host copies of the arrays
        ops.attn_prefill_ragged(gpu_ctx, cache=ops.KvCacheView(BF16, k_ptrs=ptrs, v_ptrs=ptrs), seq_lens=[16], **base)
    assert e.value.code == 1
    with pytest.raises(ShadyError) as e:      # a page size the K/V tile cannot be cut into
        ops.attn_prefill_ragged(gpu_ctx, cache=ops.KvCacheView(BF16, d, d, 0, None, None, ptrs, 48, 4), seq_lens=[16], **base)
    assert e.value.code == 2
    gpu_ctx.synchronize()


@pytest.mark.parametrize("hd", [128, 256])
def test_many_short_prompts(gpu_ctx, oracle, hd):
    """Hundreds of items of one or two K/V tiles each: the roles of a CTA run several items apart (the softmax is
    done with an item long before its epilogue starts), which is what the per-row hand-over words are numbered for."""
    rng = np.random.default_rng(77)
    lens = [int(v) for v in rng.integers(1, 200, 90)] + [130, 257, 64, 1, 128]
    _plain_case(gpu_ctx, oracle, lens, 8, 2, hd, BF16, 65, "ptrs")
